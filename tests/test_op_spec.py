"""Op-spec surface (lev_op_install_json): the reference's own op documents
and region fixtures are accepted with the reference's identities; tampered
ones are rejected.  Host-only: runs without a GPU (NULL context)."""
import ctypes as C
import hashlib
import json
import os

import pytest

from leviathan_b200 import _lib as L

HERE = os.path.dirname(os.path.abspath(__file__))
G = json.load(open(os.path.join(HERE, "golden", "op_specs.json")))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(L.LIB_PATH):
        from leviathan_b200.build import build_library

        build_library()
    return L.load()


def install(lib, doc):
    data = doc.encode() if isinstance(doc, str) else doc
    h = C.c_void_p()
    st = lib.lev_op_install_json(None, data, len(data), C.byref(h))
    return st, h


def describe(lib, h):
    kind, ident, kern = C.create_string_buffer(32), C.create_string_buffer(65), C.create_string_buffer(64)
    i, o, t, c = C.c_int64(), C.c_int64(), C.c_int(), C.c_int()
    assert lib.lev_op_describe(h, kind, C.byref(i), C.byref(o), C.byref(t), C.byref(c), ident, kern) == 0
    return kind.value.decode(), i.value, o.value, t.value, c.value, ident.value.decode(), kern.value.decode()


def test_reference_q4_ops_install_with_the_reference_identity(lib):
    assert len(G["ops"]) == 3
    for op in G["ops"]:
        st, h = install(lib, op["json"])
        assert st == 0
        kind, i, o, t, c, ident, kern = describe(lib, h)
        assert (kind, i, o, t, c) == ("q4_0.matvec", op["inDim"], op["outDim"], 2, 1)
        assert ident == op["identity"] and kern == "lev_matvec_stream"
        lib.lev_op_uninstall(None, h)


def test_reference_regions_install_and_digest(lib):
    for reg in G["regions"]:
        st, h = install(lib, reg["json"])
        assert st == 0, reg["hidden"]
        kind, i, o, t, c, ident, kern = describe(lib, h)
        assert kind == "moe.routed-region" and i == reg["hidden"] and ident == reg["graphSha256"]
        lib.lev_op_uninstall(None, h)


def _mut(doc, **kw):
    d = json.loads(doc)
    for k, v in kw.items():
        if v is KeyError:
            d.pop(k, None)
        else:
            d[k] = v
    return json.dumps(d)


def test_op_rejections(lib):
    base = G["ops"][0]["json"]
    BAD = 14  # LEV_BAD_OP_SPEC
    for bad in (
        _mut(base, schema=2), _mut(base, op="q4_0.matmul"), _mut(base, semantics="dot"), _mut(base, inDim=33),
        _mut(base, outDim=0), _mut(base, layout="col-major"), _mut(base, quant="q5_0"), _mut(base, accumulate="f16"),
        _mut(base, inputPrecision="f16"), _mut(base, view="diagonal"), _mut(base, tensor="blk.0.attn_q.weight"),
        _mut(base, representativeRows=0), _mut(base, representativeRows=5000), _mut(base, surprise=1),
        _mut(base, inDim=KeyError), _mut(base, columns=9), _mut(base, inDim="2816"), base + "x", "[1,2]", "{",
        _mut(base, inDim=(1 << 22) + 32),
    ):
        st, h = install(lib, bad)
        assert st == BAD and not h.value, bad[:80]
    st, _ = install(lib, " " * 70000)
    assert st == BAD


def test_extended_quants_and_gemm_ops(lib):
    for quant, t, blk in (("q4_k", 12, 256), ("q6_k", 14, 256)):
        doc = {"schema": 1, "op": f"{quant}.matvec", "semantics": "dot(W_row, x)", "inDim": 4096, "outDim": 12288,
               "layout": f"row-major-{quant}-blocks", "quant": quant, "accumulate": "f32", "inputPrecision": "f32", "columns": 4}
        st, h = install(lib, json.dumps(doc))
        assert st == 0
        assert describe(lib, h)[:5] == (f"{quant}.matvec", 4096, 12288, t, 4)
        lib.lev_op_uninstall(None, h)
        st, _ = install(lib, json.dumps(dict(doc, inDim=4096 + 32)))
        assert st == 14
        g = dict(doc, op=f"{quant}.gemm", inputPrecision="bf16", columns=512)
        st, h = install(lib, json.dumps(g))
        assert st == 0 and describe(lib, h)[6] == "lev_gemm_prefill"
        lib.lev_op_uninstall(None, h)


def test_region_tamper_is_rejected(lib):
    """Sources/leviathan-tests/main.swift:5733-6698: lies about topK, gelu, an extra node."""
    doc = G["regions"][0]["json"]
    for bad in (_mut(doc, topK=4), _mut(doc, geluApprox="none"), _mut(doc, gateUpOut=32), _mut(doc, stackOutputs=False),
                _mut(doc, slotOps=["a", "b", "c"]), _mut(doc, hidden=100), _mut(doc, graphSha256="0" * 64), _mut(doc, extra=1)):
        st, h = install(lib, bad)
        assert st == 14 and not h.value
    d = json.loads(doc)
    d["graph"]["nodes"].append(dict(d["graph"]["nodes"][-1], name="extra_node"))
    st, _ = install(lib, json.dumps(d))
    assert st == 14
    d = json.loads(doc)
    d["graph"]["nodes"][5]["args"], d["graph"]["nodes"][6]["args"] = d["graph"]["nodes"][6]["args"], d["graph"]["nodes"][5]["args"]
    st, _ = install(lib, json.dumps(d))
    assert st == 14


# ---- the graph walk: tampers whose digest is recomputed, so that only the structural re-derivation can catch them ----
def _canon_val(v):
    if v is None:
        return "n"
    if isinstance(v, bool):
        return "b:1" if v else "b:0"
    if isinstance(v, int):
        return f"i:{v}"
    if isinstance(v, str):
        return "s:" + v
    if isinstance(v, dict):
        assert list(v) == ["__node__"]
        return "@" + v["__node__"]
    return "l<" + ",".join(_canon_val(e) for e in v) + ">"


def _canon_meta(m):
    if m is None:
        return "n"
    out = "d<dtype:s:" + m["dtype"]
    if isinstance(m.get("items"), list):
        out += ",items:l<" + ",".join(_canon_meta(i) for i in m["items"]) + ">"
    sh = m.get("shape")
    out += ",shape:" + ("l<" + ",".join(f"i:{d}" for d in sh) + ">" if isinstance(sh, list) else "n") + ">"
    return out


def graph_digest(graph) -> str:
    """The canonical node lines of MoELowering.swift:66-168, restated for the tests."""
    lines = []
    for n in graph["nodes"]:
        kw = ",".join(f"{k}:{_canon_val(v)}" for k, v in sorted(n["kwargs"].items()))
        lines.append(f'{n["name"]}|{n["op"]}|{n["target"]}|{_canon_val(n["args"])}|d<{kw}>|{_canon_meta(n.get("meta"))}\n')
    payload = "".join(lines) + "inputs|" + _canon_val(graph["inputs"]) + "\noutputs|" + _canon_val(graph["outputs"])
    return hashlib.sha256(payload.encode()).hexdigest()


def _retamper(doc, edit):
    d = json.loads(doc)
    edit(d["graph"]["nodes"], d)
    d["graphSha256"] = graph_digest(d["graph"])
    return json.dumps(d)


def _message(lib, doc):
    """install with a context-free call and return (status, accepted handle)"""
    st, h = install(lib, doc)
    return st, h


def test_the_test_digest_reproduces_the_reference_digests():
    for reg in G["regions"]:
        assert graph_digest(json.loads(reg["json"])["graph"]) == reg["graphSha256"]


def _by_target(nodes, target):
    return [n for n in nodes if n["target"] == target]


def test_graph_walk_rejects_restructured_graphs_with_a_matching_digest(lib):
    """Sources/leviathan-tests/main.swift:5778-5820 (swapped getitems, gelu approximate=none, an extra node) and the
    other structural guards of MoERegionGraphWalk.walk, each with graphSha256 recomputed for the edited graph."""
    doc = G["regions"][0]["json"]
    ok, h = install(lib, _retamper(doc, lambda nodes, d: None))
    assert ok == 0
    lib.lev_op_uninstall(None, h)

    def swap_getitems(nodes, d):
        for n in _by_target(nodes, "operator.getitem"):
            n["args"][1] = 1 - n["args"][1]

    def gelu_none(nodes, d):
        for n in _by_target(nodes, "aten.gelu.default"):
            n["kwargs"] = {"approximate": "none"}

    def extra_sin(nodes, d):
        nodes.append({"name": "extra_sin", "op": "call_function", "target": "aten.sin.default", "args": [{"__node__": nodes[3]["name"]}],
                      "kwargs": {}, "meta": None})

    def slot_order(nodes, d):  # slot 0 selects expert row 1 and slot 1 row 0
        sel = [n for n in _by_target(nodes, "aten.select.int") if n["args"][0]["__node__"] == "gu_weights"]
        sel[0]["args"][2], sel[1]["args"][2] = sel[1]["args"][2], sel[0]["args"][2]

    def shared_select(nodes, d):  # two slots read the same down slice node
        lin = [n for n in _by_target(nodes, "aten.linear.default") if n["args"][0]["__node__"].startswith("mul")]
        lin[1]["args"][1] = dict(lin[0]["args"][1])

    def private_x(nodes, d):  # a slot's gate_up projection reads something other than the shared input
        lin = [n for n in _by_target(nodes, "aten.linear.default") if n["args"][0]["__node__"] == "x"]
        lin[1]["args"][0] = {"__node__": "gu_weights"}

    def bias(nodes, d):
        _by_target(nodes, "aten.linear.default")[0]["args"].append({"__node__": "x"})

    def split_dim(nodes, d):
        _by_target(nodes, "aten.split.Tensor")[0]["args"][2] = 1

    def split_size(nodes, d):
        _by_target(nodes, "aten.split.Tensor")[1]["args"][1] = 16

    def meta_shape(nodes, d):
        _by_target(nodes, "aten.mul.Tensor")[0]["meta"]["shape"] = [1, 64]

    def meta_dtype(nodes, d):
        nodes[0]["meta"]["dtype"] = "float16"

    def stack_dim(nodes, d):
        _by_target(nodes, "aten.stack.default")[0]["args"].append(1)

    def stack_short(nodes, d):
        _by_target(nodes, "aten.stack.default")[0]["args"][0].pop()

    def batch_two(nodes, d):
        nodes[0]["meta"]["shape"][0] = 2

    def placeholder_kwargs(nodes, d):
        nodes[0]["kwargs"] = {"a": 1}

    def node_kind(nodes, d):
        nodes[3]["op"] = "call_method"

    def duplicate_name(nodes, d):
        nodes[4]["name"] = nodes[3]["name"]

    def inputs_order(nodes, d):
        d["graph"]["inputs"] = ["gu_weights", "x", "down_weights"]

    def mul_is_add(nodes, d):
        _by_target(nodes, "aten.mul.Tensor")[0]["target"] = "aten.add.Tensor"

    def huge_dim(nodes, d):
        nodes[1]["meta"]["shape"][1] = 1 << 40

    edits = [swap_getitems, gelu_none, extra_sin, slot_order, shared_select, private_x, bias, split_dim, split_size, meta_shape, meta_dtype,
             stack_dim, stack_short, batch_two, placeholder_kwargs, node_kind, duplicate_name, inputs_order, mul_is_add, huge_dim]
    for e in edits:
        st, h = install(lib, _retamper(doc, e))
        assert st == 14 and not h.value, e.__name__

    # accepted spellings of the same graph: stack's dim as a second operand or as a keyword, a null bias operand
    def dim_operand(nodes, d):
        _by_target(nodes, "aten.stack.default")[0]["args"].append(0)

    def dim_keyword(nodes, d):
        _by_target(nodes, "aten.stack.default")[0]["kwargs"] = {"dim": 0}

    def null_bias(nodes, d):
        for n in _by_target(nodes, "aten.linear.default"):
            n["args"].append(None)

    for e in (dim_operand, dim_keyword, null_bias):
        st, h = install(lib, _retamper(doc, e))
        assert st == 0, e.__name__
        lib.lev_op_uninstall(None, h)


def test_declared_dims_must_agree_with_the_graph(lib):
    """main.swift:5778-5781: the scalar fields lie, the graph (and its digest) are untouched."""
    big = [r for r in G["regions"] if r["hidden"] != 96]
    doc = (big[0] if big else G["regions"][0])["json"]
    d = json.loads(doc)
    for field, value in (("topK", d["topK"] - 1), ("hidden", d["hidden"] - 32), ("expertIntermediate", d["expertIntermediate"] + 32)):
        e = dict(d)
        e[field] = value
        if field == "expertIntermediate":
            e["gateUpOut"] = 2 * value
        st, h = install(lib, json.dumps(e))
        assert st == 14 and not h.value, field
