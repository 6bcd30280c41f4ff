"""GGUF container reader (lev_gguf_*): accepted files, every rejection of the
reference's reader (Sources/LeviathanCore/GGUF.swift:191-362; its tests in
Tests/LeviathanCoreTests/GGUFTests.swift cover the same cases), and upload of a
quantized tensor from a file."""
import struct

import numpy as np
import pytest

from leviathan_b200 import GGUFFile, LevError, GGML_Q4_0, GGML_Q4_K, GGML_Q6_K
from leviathan_b200 import quant

from gguf_build import ARR, F32, F64, I32, STR, U32, U64, as_bytes, build, kv


def _q(ty, seed, rows, cols):
    return quant.quantized_normal(ty, seed, rows, cols).numpy()


def _model_tensors():
    return [
        ("blk.0.ffn_gate.weight", [256, 48], GGML_Q4_K, as_bytes(_q(GGML_Q4_K, 1, 48, 256))),
        ("blk.0.ffn_down.weight", [512, 32], GGML_Q6_K, as_bytes(_q(GGML_Q6_K, 2, 32, 512))),
        ("blk.0.attn_q.weight", [64, 16], GGML_Q4_0, as_bytes(_q(GGML_Q4_0, 3, 16, 64))),
        ("blk.0.ffn_gate_exps.weight", [64, 16, 4], GGML_Q4_0, as_bytes(_q(GGML_Q4_0, 4, 64, 64))),
        ("output_norm.weight", [64], 0, as_bytes(np.arange(64, dtype=np.float32))),
    ]


META = [kv("general.architecture", STR, "gemma4"), kv("gemma4.block_count", U32, 1),
        kv("gemma4.context_length", U64, 8192), kv("gemma4.rope.freq_base", F32, 10000.0),
        kv("gemma4.scale", F64, 0.125), kv("gemma4.signed", I32, -5),
        kv("tokenizer.ggml.tokens", ARR, ["a", "bc", ""], STR), kv("tokenizer.ggml.scores", ARR, [0.5, -1.0], F32)]


def expect(status_name, blob):
    with pytest.raises(LevError) as e:
        GGUFFile(blob)
    assert e.value.name == status_name, (e.value.name, e.value.message)
    return e.value


@pytest.mark.parametrize("version", [2, 3])
@pytest.mark.parametrize("alignment", [None, 64, 4096])
def test_directory_and_metadata(version, alignment):
    tensors = _model_tensors()
    blob = build(tensors, META, version=version, alignment=alignment)
    with GGUFFile(blob) as g:
        assert g.version == version and g.tensor_count == len(tensors)
        assert g.alignment == (alignment or 32) and g.data_offset % g.alignment == 0
        assert g.metadata_count == len(META) + (alignment is not None)
        for i, (name, dims, ty, data) in enumerate(tensors):
            t = g.tensor(name)
            assert t == g.tensor(i)
            assert (t["name"], t["dims"], t["ggml_type"], t["n_bytes"]) == (name, dims, ty, len(data))
            assert t["file_offset"] % g.alignment == 0
            assert blob[t["file_offset"]:t["file_offset"] + t["n_bytes"]] == data
            assert g.tensor_bytes(name).tobytes() == data
        assert g.meta_string("general.architecture") == "gemma4"
        assert g.meta_uint("gemma4.block_count") == 1 and g.meta_uint("gemma4.context_length") == 8192
        assert g.meta_uint("gemma4.signed") == 0  # negative integers read as 0
        assert g.meta_array("tokenizer.ggml.tokens") == ["a", "bc", ""]
        assert g.meta_array("tokenizer.ggml.scores") == [0.5, -1.0]
        assert g.meta_float("gemma4.rope.freq_base") == 10000.0 and g.meta_float("gemma4.scale") == 0.125
        for bad in ("absent.key", "general.architecture"):
            with pytest.raises(LevError) as e:
                g.meta_uint(bad)
            assert e.value.name == "missing"
        with pytest.raises(LevError) as e:
            g.tensor("no.such.tensor")
        assert e.value.name == "missing"


def test_open_maps_a_file(tmp_path):
    tensors = _model_tensors()
    p = tmp_path / "m.gguf"
    p.write_bytes(build(tensors, META))
    with GGUFFile(str(p)) as g:
        assert [t["name"] for t in g.tensors()] == [t[0] for t in tensors]
        assert g.tensor_bytes("blk.0.ffn_down.weight").tobytes() == tensors[1][3]
    with pytest.raises(LevError):
        GGUFFile(str(tmp_path / "absent.gguf"))
    (tmp_path / "short.gguf").write_bytes(b"GGUF")
    with pytest.raises(LevError) as e:
        GGUFFile(str(tmp_path / "short.gguf"))
    assert e.value.name == "truncated"


def test_empty_container():
    with GGUFFile(build([], [])) as g:
        assert g.tensor_count == 0 and g.metadata_count == 0 and g.data_offset == 32


def test_reads_what_gguf_py_writes(tmp_path):
    gguf = pytest.importorskip("gguf")
    p = str(tmp_path / "w.gguf")
    w = gguf.GGUFWriter(p, "llama")
    w.add_uint32("llama.block_count", 2)
    q4 = _q(GGML_Q4_0, 5, 16, 64).reshape(16, -1)
    q6 = _q(GGML_Q6_K, 6, 8, 256).reshape(8, -1)
    w.add_tensor("a.weight", q4, raw_dtype=gguf.GGMLQuantizationType.Q4_0)
    w.add_tensor("b.weight", q6, raw_dtype=gguf.GGMLQuantizationType.Q6_K)
    w.add_tensor("n.weight", np.ones(64, np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with GGUFFile(p) as g:
        assert g.version == 3 and g.tensor_count == 3 and g.meta_uint("llama.block_count") == 2
        assert g.meta_string("general.architecture") == "llama"
        a, b = g.tensor("a.weight"), g.tensor("b.weight")
        assert a["dims"] == [64, 16] and a["ggml_type"] == GGML_Q4_0
        assert b["dims"] == [256, 8] and b["ggml_type"] == GGML_Q6_K
        assert g.tensor_bytes("a.weight").tobytes() == q4.tobytes()
        assert g.tensor_bytes("b.weight").tobytes() == q6.tobytes()


# ---- rejections ----------------------------------------------------------

def test_rejects_bad_magic_and_version():
    t = _model_tensors()[:1]
    expect("badMagic", build(t, magic=b"GGML"))
    expect("unsupportedVersion", build(t, version=1))
    expect("unsupportedVersion", build(t, version=4))
    expect("truncated", b"GGUF\x03\0\0")


def test_rejects_truncation_everywhere():
    blob = build(_model_tensors()[:2], META)
    with GGUFFile(blob) as g:
        header_end = g.data_offset
    for cut in list(range(4, header_end - 32, 7)):
        with pytest.raises(LevError) as e:
            GGUFFile(blob[:cut])
        assert e.value.name in ("truncated", "dataBeyondEndOfFile"), (cut, e.value.name)
    expect("dataBeyondEndOfFile", blob[:-1])


def test_rejects_implausible_counts_and_lengths():
    t = _model_tensors()[:1]
    expect("truncated", build(t, counts=(100001, 0)))
    expect("truncated", build(t, counts=(1, 1 << 40)))
    with pytest.raises(LevError):  # promises more entries than the file has: tensor bytes read as directory
        GGUFFile(build(t, counts=(5, 0)))
    long_key = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", (1 << 20) + 1) + b"x" * 64
    expect("truncated", long_key)
    huge_array = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IIQ", 9, 4, 10_000_001)
    expect("truncated", huge_array)
    expect("truncated", build([], [kv("k", U32, 1), kv("k", U32, 2)]))  # duplicate key


def test_rejects_unknown_value_types():
    head = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k"
    expect("unknownValueType", head + struct.pack("<I", 13) + b"\0" * 16)
    expect("unknownValueType", head + struct.pack("<IIQ", 9, 9, 0) + b"\0" * 16)  # array of arrays
    expect("unknownValueType", head + struct.pack("<IIQ", 9, 77, 1) + b"\0" * 16)


def test_rejects_bad_alignment():
    expect("truncated", build([], alignment=0))
    expect("truncated", build([], alignment=(1 << 20) + 1))


def test_rejects_bad_tensors():
    q = as_bytes(_q(GGML_Q4_0, 7, 4, 64))
    expect("badTensor", build([("t", [], GGML_Q4_0, q)]))                      # no dimensions
    expect("badTensor", build([("t", [64, 1, 1, 1, 4], GGML_Q4_0, q)]))        # five dimensions
    expect("badTensor", build([("t", [64, 0], GGML_Q4_0, q)]))                 # zero dimension
    expect("badTensor", build([("t", [48, 4], GGML_Q4_0, q)]))                 # rows not whole blocks
    expect("badTensor", build([("t", [64, 4], GGML_Q4_0, q)], offsets=[8]))    # misaligned offset
    expect("badTensor", build([("t", [64, 4], GGML_Q4_0, q), ("t", [64, 4], GGML_Q4_0, q)]))  # duplicate name
    expect("badTensor", build([("a", [64, 4], GGML_Q4_0, q), ("b", [64, 4], GGML_Q4_0, q)], offsets=[0, 32]))  # overlap
    expect("badTensor", build([("a", [64, 4], GGML_Q4_0, q), ("b", [64, 4], GGML_Q4_0, q)], offsets=[0, 0]))
    expect("unsupportedTensorType", build([("t", [64, 4], 3, q)]))             # Q4_1 is not sized here
    expect("unsupportedTensorType", build([("t", [64, 4], 9999, q)]))
    expect("dataBeyondEndOfFile", build([("t", [64, 8], GGML_Q4_0, q)]))       # claims twice its bytes
    expect("dataBeyondEndOfFile", build([("t", [64, 4], GGML_Q4_0, q)], offsets=[1 << 40]))
    e = expect("integerOverflow", build([("t", [1 << 30, 1 << 30], GGML_Q4_0, q)]))
    assert "element count" in e.message
    expect("badTensor", build([("t", [(1 << 40) + 32, 1], GGML_Q4_0, q)]))     # one dimension beyond the cap
    expect("integerOverflow", build([("t", [64, 4], GGML_Q4_0, q)], offsets=[(1 << 63) + 32]))


# ---- upload from a file ----------------------------------------------------

@pytest.mark.gpu
def test_upload_from_file_matches_oracle(tmp_path):
    import leviathan_b200 as lev
    from oracle import oracle as O

    tensors = _model_tensors()
    p = tmp_path / "m.gguf"
    p.write_bytes(build(tensors, META, alignment=64))
    with lev.Context() as ctx, GGUFFile(str(p)) as g:
        for name, dims, ty, data in tensors[:4]:
            w = g.upload(ctx, name)
            rows = dims[1] * (dims[2] if len(dims) == 3 else 1)
            assert (w.ggml_type, w.rows, w.cols) == (ty, rows, dims[0])
            blocks = np.frombuffer(data, np.uint8)
            x = quant.normal(11, (dims[0],), 1.0)
            x = x.reshape(1, -1).astype(np.float32)
            got = ctx.matvec(w, x)
            assert O.max_rel_err(got[0], O.matvec_f64(ty, blocks, rows, dims[0], x[0])) < 1e-4
            ref = O.dequantize_rows(ty, blocks, rows, dims[0])
            assert np.array_equal(ctx.dequantize(w).view(np.uint32), ref.view(np.uint32))
            w.free()
        with pytest.raises(LevError) as e:
            g.upload(ctx, "output_norm.weight")
        assert e.value.name == "unsupportedTensorType"
        with pytest.raises(LevError) as e:
            g.upload(ctx, "absent")
        assert e.value.name == "missing"


def test_reference_known_container_and_messages():
    """The hand-built container and the rejection cases of the reference's own test
    runner (Sources/leviathan-tests/main.swift:508-640), rebuilt from their description."""
    raw = lambda *parts: b"GGUF" + b"".join(parts)  # noqa: E731
    u32 = lambda v: struct.pack("<I", v)  # noqa: E731
    u64 = lambda v: struct.pack("<Q", v)  # noqa: E731
    s = lambda t: u64(len(t)) + t.encode()  # noqa: E731
    pad = lambda b: b + b"\0" * (-len(b) % 32)  # noqa: E731
    tinfo = lambda name, d0, d1, ty, off: s(name) + u32(2) + u64(d0) + u64(d1) + u32(ty) + u64(off)  # noqa: E731

    head = pad(raw(u32(3), u64(1), u64(2), s("general.alignment"), u32(4), u32(32),
                   s("gemma4.context_length"), u32(10), u64(262144), tinfo("test_tensor", 32, 4, 2, 0)))
    blob = head + b"\x7f" * 72
    with GGUFFile(blob) as g:
        assert g.version == 3 and g.tensor_count == 1
        assert g.meta_uint("general.alignment") == 32 and g.meta_uint("gemma4.context_length") == 262144
        t = g.tensor("test_tensor")
        assert t["dims"] == [32, 4] and t["ggml_type"] == 2
        assert (t["file_offset"], t["n_bytes"]) == (len(blob) - 72, 72)
        with pytest.raises(LevError) as e:
            g.tensor("absent")
        assert e.value.name == "missing"

    expect("badMagic", bytes([0x47, 0x47, 0x55, 0x58, 3, 0, 0, 0, 0, 0, 0, 0]))
    expect("truncated", raw(u32(2), b"\0\0\0\0"))
    assert expect("truncated", raw(u32(3), u64(0), u64(2**64 - 1))).message == "implausible tensor/kv counts"
    e = expect("truncated", raw(u32(3), u64(0), u64(1), s("k"), u32(8), u64(2**64 - 1)))
    assert "string length beyond cap" in e.message
    expect("unknownValueType", raw(u32(3), u64(0), u64(1), s("k"), u32(9), u32(9), u64(0)))
    assert expect("truncated", raw(u32(3), u64(0), u64(1), s("k"), u32(9), u32(0), u64(2**64 - 1))).message == "array too long"
    assert expect("badTensor", raw(u32(3), u64(1), u64(0), tinfo("t", 0, 4, 2, 0))).message == "tensor t: invalid dimension"
    assert expect("badTensor", raw(u32(3), u64(1), u64(0), tinfo("t", 2**64 - 1, 1, 2, 0))).message == "tensor t: invalid dimension"
    e = expect("badTensor", pad(raw(u32(3), u64(1), u64(0), tinfo("t", 31, 1, 2, 0))) + b"\0" * 18)
    assert "not a multiple of the block" in e.message
    expect("unsupportedTensorType", pad(raw(u32(3), u64(1), u64(0), tinfo("t", 32, 1, 3, 0))) + b"\0" * 20)
    expect("dataBeyondEndOfFile", pad(raw(u32(3), u64(1), u64(0), tinfo("t", 32, 1, 2, 0))))
    e = expect("badTensor", pad(raw(u32(3), u64(1), u64(0), tinfo("t", 32, 1, 2, 3))) + b"\0" * 36)
    assert e.message == "tensor t: offset 3 misaligned"
    e = expect("badTensor", pad(raw(u32(3), u64(2), u64(0), tinfo("t1", 32, 1, 2, 0), tinfo("t2", 32, 1, 2, 0))) + b"\0" * 18)
    assert e.message == "tensor t2 overlaps t1"
    e = expect("badTensor", pad(raw(u32(3), u64(2), u64(0), tinfo("t", 32, 1, 2, 0), tinfo("t", 32, 1, 2, 0))) + b"\0" * 36)
    assert e.message == "duplicate tensor name t"
    # arrays with the real element layout, followed by more metadata: the cursor lands exactly
    arr = raw(u32(3), u64(0), u64(3), s("names"), u32(9), u32(8), u64(2), s("alpha"), s("beta"),
              s("ids"), u32(9), u32(5), u64(3), struct.pack("<iii", 1, -2, 3), s("after"), u32(4), u32(77))
    with GGUFFile(arr) as g:
        assert g.metadata_count == 3 and g.meta_uint("after") == 77
        assert g.meta_array("names") == ["alpha", "beta"] and g.meta_array("ids") == [1, -2, 3]
        with pytest.raises(LevError):
            g.meta_array("after")
    # Q6_K geometry: a 256 x 2 tensor is exactly 2 * 210 bytes
    with GGUFFile(pad(raw(u32(3), u64(1), u64(0), tinfo("t", 256, 2, 14, 0))) + b"\0" * 420) as g:
        assert g.tensor("t")["n_bytes"] == 420
    # an aligned offset near the top of the signed range fails through the checked path
    expect("dataBeyondEndOfFile", pad(raw(u32(3), u64(1), u64(0), tinfo("t", 32, 1, 2, (2**63 - 1) - (2**63 - 1) % 32))))


def _moe_file(experts=8, hidden=96, inter=32, top_k=3, layers=2, seed=21, **overrides):
    """A two-layer model file holding only the routed-expert tensors (tail-region shape)."""
    rng = np.random.default_rng(seed)
    tensors, per_layer = [], []
    for layer in range(layers):
        gu = _q(GGML_Q4_0, seed + 10 * layer, experts * 2 * inter, hidden)
        dn = _q(GGML_Q4_0, seed + 10 * layer + 1, experts * hidden, inter)
        rw = (rng.standard_normal((experts, hidden)) * 0.02).astype(np.float32)
        per_layer.append((rw, gu, dn))
        tensors += [(f"blk.{layer}.ffn_gate_up_exps.weight", [hidden, 2 * inter, experts], GGML_Q4_0, as_bytes(gu)),
                    (f"blk.{layer}.ffn_down_exps.weight", [inter, hidden, experts], GGML_Q4_0, as_bytes(dn)),
                    (f"blk.{layer}.ffn_gate_inp.weight", [hidden, experts], 0, as_bytes(rw))]
    vals = dict(block_count=layers, expert_count=experts, expert_used_count=top_k, embedding_length=hidden,
                expert_feed_forward_length=inter)
    vals.update(overrides)
    meta = [kv("general.architecture", STR, "gemma4")] + [kv(f"gemma4.{k}", U32, v) for k, v in vals.items() if v is not None]
    return build(tensors, meta), per_layer


@pytest.mark.gpu
def test_moe_layer_from_file_matches_direct_upload(tmp_path):
    import leviathan_b200 as lev

    experts, hidden, inter, top_k = 8, 96, 32, 3
    blob, per_layer = _moe_file(experts, hidden, inter, top_k)
    p = tmp_path / "moe.gguf"
    p.write_bytes(blob)
    x = quant.normal(5, (7, hidden), 1.0).astype(np.float32)
    with lev.Context() as ctx, GGUFFile(str(p)) as g:
        for layer, (rw, gu, dn) in enumerate(per_layer):
            direct = ctx.moe_upload(rw, gu, dn, experts, hidden, inter)
            from_file, k = g.moe_upload(ctx, layer)
            assert k == top_k and (from_file.experts, from_file.hidden, from_file.inter) == (experts, hidden, inter)
            a, ia, wa = ctx.moe_layer(direct, x, top_k, want_routing=True)
            b, ib, wb = ctx.moe_layer(from_file, x, top_k, want_routing=True)
            assert np.array_equal(ia, ib) and np.array_equal(wa.view(np.uint32), wb.view(np.uint32))
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
            direct.free()
            from_file.free()
        # a resident window of experts (expert parallel): slices [2, 6) of the same tensors
        part, _ = g.moe_upload(ctx, 1, local_first=2, local_count=4)
        assert (part.local_first, part.local_count) == (2, 4)
        part.free()
        for bad_layer in (-1, 2):
            with pytest.raises(LevError) as e:
                g.moe_upload(ctx, bad_layer)
            assert e.value.name == "badDimensions"
        with pytest.raises(LevError) as e:
            g.moe_upload(ctx, 0, local_first=6, local_count=4)
        assert e.value.name == "badDimensions"
    with lev.Context() as ctx:
        for overrides, name in [(dict(expert_count=None), "missing"), (dict(expert_used_count=9), "badDimensions"),
                                (dict(embedding_length=64), "badDimensions"), (dict(expert_feed_forward_length=64), "badDimensions"),
                                (dict(expert_count=16), "badDimensions"), (dict(embedding_length=0), "badDimensions")]:
            with GGUFFile(_moe_file(**overrides)[0]) as g, pytest.raises(LevError) as e:
                g.moe_upload(ctx, 0)
            assert e.value.name == name, (overrides, e.value.name)
        blob2, _ = _moe_file(layers=1)
        with GGUFFile(blob2.replace(b"blk.0.ffn_gate_inp.weight", b"blk.0.ffn_gate_xxx.weight")) as g, pytest.raises(LevError) as e:
            g.moe_upload(ctx, 0)
        assert e.value.name == "missing"
