"""Generates tests/golden/op_specs.json from the reference's own Python
op-spec frontends (run where the reference tree is mounted):

  * the three shipped q4_0.matvec op models, captured with the reference's
    Q4MatvecOp.to_json / check_op (tools/q4_lower/q4_op_model.py), with the
    identity the Swift side computes for them (SHA-256 of the sorted-keys
    compact JSON, absent optionals omitted; Q4Lowering.swift:176-181);
  * the two routed-MoE region documents the reference's tests hold
    (tools/moe_lower/fixtures/*.json), whose graphSha256 is the golden value
    for the canonical graph digest (MoELowering.swift:66-168).

Usage: python tests/golden/make_op_fixtures.py /path/to/reference
"""
import hashlib
import importlib.util
import json
import os
import sys

if len(sys.argv) != 2:
    sys.exit(__doc__)
ref = sys.argv[1]
q4 = os.path.join(ref, "tools", "q4_lower")
sys.path.insert(0, q4)
from q4_op_model import Q4MatvecOp, check_op  # noqa: E402

ops = []
for name in ("model_q4_expert_gu.py", "model_q4_expert_dn.py", "model_q4_attn_output.py"):
    spec = importlib.util.spec_from_file_location("user_op_model", os.path.join(q4, name))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    built = mod.build()
    obj = built.to_json() if isinstance(built, Q4MatvecOp) else built
    check_op(obj)
    canon = json.dumps({k: v for k, v in obj.items() if v is not None}, sort_keys=True, separators=(",", ":"),
                       ensure_ascii=False)
    ops.append({"json": json.dumps(obj, sort_keys=True, ensure_ascii=False),
                "identity": hashlib.sha256(canon.encode()).hexdigest(),
                "inDim": obj["inDim"], "outDim": obj["outDim"]})
regions = []
for name in ("tail-region.json", "gemma4-26b-region.json"):
    doc = json.load(open(os.path.join(ref, "tools", "moe_lower", "fixtures", name)))
    regions.append({"json": json.dumps(doc, separators=(",", ":")), "graphSha256": doc["graphSha256"],
                    "hidden": doc["hidden"], "expertIntermediate": doc["expertIntermediate"], "topK": doc["topK"]})
out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "op_specs.json")
json.dump({"ops": ops, "regions": regions}, open(out, "w"), indent=0)
print(out, len(ops), len(regions))
