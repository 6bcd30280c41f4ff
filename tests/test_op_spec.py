"""Op-spec surface (lev_op_install_json): the reference's own op documents
and region fixtures are accepted with the reference's identities; tampered
ones are rejected.  Host-only: runs without a GPU (NULL context)."""
import ctypes as C
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
