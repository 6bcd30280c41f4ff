"""The oracle against every known-answer vector the reference's own tests
hold for this path.  Each test names the reference test it restates."""
import math

import numpy as np
import pytest

from leviathan_b200 import quant as Q
from oracle import oracle as O


# ---- f16 (rust/crates/lev-cpu/src/lib.rs:411-419, :559-566) ----
def test_half_conversion_known_values():
    assert O.f16_to_f64(0x3C00) == 1.0
    assert O.f16_to_f64(0xC000) == -2.0
    assert O.f16_to_f64(0x0001) == 2.0 ** -24
    assert O.f16_to_f64(0x7BFF) == 65504.0
    assert O.f16_to_f64(0x7C00) == math.inf
    assert math.isnan(O.f16_to_f64(0x7E00))
    assert O.f16_to_f64(0x0000) == 0.0


def test_f16_round_trips_and_rounds_to_even():
    for h in [0, 1, 0x3C00, 0xBC00, 0x7BFF, 0x0400, 0x03FF, 0x3555]:
        assert O.f32_to_f16_bits(O.f16_to_f32(h)) == h
    assert O.f32_to_f16_bits(1.0 + 1.0 / 2048.0) == 0x3C00
    assert O.f32_to_f16_bits(1.0 + 3.0 / 2048.0) == 0x3C02
    assert O.f32_to_f16_bits(1e9) == 0x7C00
    assert O.f32_to_f16_bits(-0.0) == 0x8000


def test_f16_matches_numpy_for_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float64)
    got = np.array([O.f16_to_f64(int(b)) for b in bits])
    finite = np.isfinite(ref)
    assert np.array_equal(got[finite], ref[finite])
    assert np.array_equal(np.isnan(got), np.isnan(ref))


def test_bf16_rounding_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    v = rng.standard_normal(4096).astype(np.float32)
    ref = torch.from_numpy(v).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    got = np.array([O.f32_to_bf16_bits(float(a)) for a in v], dtype=np.uint16)
    assert np.array_equal(got, ref)


# ---- Q4_0 (Sources/leviathan-tests/main.swift:703-746) ----
def test_q4_0_known_block():
    block = [0x00, 0x3C] + list(range(16))
    expected = [float(l) - 8 for l in range(16)] + [-8.0] * 16
    got = O.q4_0_decode_block(block)
    assert got.tolist() == expected
    half = list(block)
    half[1] = 0x38
    assert O.q4_0_decode_block(half)[0] == 0.5 * -8
    inf = list(block)
    inf[1] = 0x7C
    with pytest.raises(O.OracleError) as e:
        O.q4_0_decode_block(inf)
    assert e.value.name == "nonFiniteScale"


def test_q4_0_streaming_matvec_two_rows():
    w = [0x00, 0x3C] + [0] * 16 + [0x00, 0xBC] + [0] * 16
    x = O.seeded_input_swift(32, 7)
    sum_x = np.float32(0)
    for v in x:
        sum_x = np.float32(sum_x + v)
    y = O.q4_0_matvec_f32(w, 2, 32, x)
    assert y.shape == (2,)
    assert abs(y[0] - (-8 * sum_x)) < 1e-3
    assert abs(y[1] - (8 * sum_x)) < 1e-3
    bad = x.copy()
    bad[0] = np.nan
    with pytest.raises(O.OracleError) as e:
        O.q4_0_matvec_f32(w, 2, 32, bad)
    assert e.value.name == "nonFiniteInput"


def test_q4_0_geometry_rejections():
    # Sources/leviathan-tests/main.swift:778-796
    with pytest.raises(O.OracleError) as e:
        O.q4_0_matvec_f32([], 8, 33, [])
    assert e.value.name == "badDimensions"
    with pytest.raises(O.OracleError) as e:
        O.q4_0_matvec_f32([], 8, 32, [])
    assert e.value.name == "badDimensions"
    with pytest.raises(O.OracleError) as e:
        O.q4_0_matvec_f32([0] * (8 * 18), 8, 32, [0, 0, 0])
    assert e.value.name == "wrongInputCount"


def _swift_random_q4_0(rows, bpr, seed):
    # Sources/leviathan-tests/main.swift:754-761
    r = O.SplitMix64(seed)
    out = bytearray()
    for _ in range(rows * bpr):
        scale = np.float16(np.float32(r.uniform_swift()) * np.float32(2) - np.float32(1))
        bits = int(scale.view(np.uint16))
        out += bytes([bits & 0xFF, bits >> 8])
        for _ in range(16):
            out.append(r.next() & 0xFF)
    return np.frombuffer(bytes(out), np.uint8)


def test_q4_0_f32_within_gate_of_f64_on_reference_generator():
    # statistical gate of Sources/leviathan-tests/main.swift:748-773
    w = _swift_random_q4_0(128, 8, 99)
    x = O.seeded_input_swift(256, 101)
    y32 = O.q4_0_matvec_f32(w, 128, 256, x)
    y64 = O.q4_0_matvec_f64(w, 128, 256, x)
    assert O.max_rel_err(y32, y64) < 1e-4
    assert O.max_rel_err(O.q4_0_matvec_f32_interleaved(w, 128, 256, x), y64) < 1e-4
    # the double-input MoE form agrees with the float-input gate oracle to 1e-12
    y64b = O.q4_0_matvec_f64_dx(w, 0, 128, 256, x.astype(np.float64))
    assert np.max(np.abs(y64b - y64) / np.maximum(1, np.abs(y64))) < 1e-12


# ---- Q4_K (rust/crates/lev-cpu/src/lib.rs:421-493) ----
def test_q4_k_scale_min_round_trip():
    r = O.SplitMix64(7)
    for _ in range(2000):
        sc, mn = [], []
        for _j in range(8):
            sc.append(r.next() % 64)
            mn.append(r.next() % 64)
        packed = O.q4_k_pack_scale_min(sc, mn)
        for j in range(8):
            assert O.q4_k_unpack_scale_min(j, packed) == (sc[j], mn[j])


def test_q4_k_hand_computed_block():
    block = np.zeros(144, np.uint8)
    block[0:2] = [0x00, 0x3C]
    block[2:4] = [0x00, 0x38]
    block[4:16] = O.q4_k_pack_scale_min([1] * 8, [2] * 8)
    block[16:] = 0x21
    f32 = O.q4_k_dequant_block_f32(block)
    f64 = O.q4_k_dequant_block_f64(block)
    for chunk in range(4):
        assert np.all(f64[chunk * 64: chunk * 64 + 32] == 0.0)
        assert np.all(f64[chunk * 64 + 32: chunk * 64 + 64] == 1.0)
        assert np.all(f32[chunk * 64: chunk * 64 + 32] == 0.0)
        assert np.all(f32[chunk * 64 + 32: chunk * 64 + 64] == 1.0)


def _rust_random_q4_k(r, n):
    halves = [0x2E66, 0x3000, 0x3266, 0x2800, 0x1C00, 0x3400]
    out = bytearray()
    for _ in range(n):
        for _ in range(2):
            h = halves[r.next() % 6]
            out += bytes([h & 0xFF, h >> 8])
        for _ in range(140):
            out.append(r.next() & 0xFF)
    return np.frombuffer(bytes(out), np.uint8)


def test_q4_k_f32_matches_f64_oracle():
    r = O.SplitMix64(42)
    rows, cols = 16, 1024
    w = _rust_random_q4_k(r, rows * cols // 256)
    x = np.array([r.signed_unit_rust() for _ in range(cols)], np.float32)
    got = O.q4_k_matvec_f32(w, rows, cols, x)
    ref = O.q4_k_matvec_f64(w, rows, cols, x)
    assert O.max_rel_err(got, ref) < 1e-4


def test_q4_k_shape_errors():
    x = np.zeros(256, np.float32)
    with pytest.raises(O.OracleError):
        O.q4_k_matvec_f32([], 1, 100, x[:100])
    with pytest.raises(O.OracleError):
        O.q4_k_matvec_f32([0] * 10, 1, 256, x)
    with pytest.raises(O.OracleError) as e:
        O.q4_k_matvec_f32([0] * 144, 1, 256, x[:10])
    assert e.value.name == "wrongInputCount"


def test_max_rel_err_gate():
    assert O.max_rel_err([np.nan], [0.0]) == math.inf
    assert O.max_rel_err([1.0], [math.inf]) == math.inf
    assert O.max_rel_err([1.0, 2.0], [1.0]) == math.inf
    assert O.max_rel_err([], []) == math.inf
    assert O.max_rel_err([1.0], [1.0]) == 0.0
    # Sources/leviathan-tests/main.swift:8947-8951
    assert O.max_rel_err([1001.0], [1000.0]) == 0.001
    assert O.max_rel_err([0.5], [0.0]) == 0.5


# ---- Q6_K (Sources/leviathan-tests/main.swift:993-1026, :1087-1123;
#      rust/crates/lev-cpu/src/lib.rs:496-541) ----
def test_q6_k_known_block_swift():
    block = np.zeros(210, np.uint8)
    block[208], block[209] = 0x00, 0x3C
    block[192:208] = 1
    block[0] = 0x21
    block[128] = 0x03
    v = O.q6_k_decode_block(block)
    assert v.shape == (256,)
    assert v[0] == 17 and v[32] == -32 and v[64] == -30 and v[96] == -32 and v[1] == -32
    block[193] = 2
    assert O.q6_k_decode_block(block)[20] == 2 * -32
    block[209] = 0x7C
    with pytest.raises(O.OracleError) as e:
        O.q6_k_decode_block(block)
    assert e.value.name == "nonFiniteScale"


def test_q6_k_minus_315_dot():
    block = np.zeros(210, np.uint8)
    block[208], block[209] = 0x00, 0x3C
    block[192] = 3
    block[193] = 0xFD
    block[196] = 2
    block[200] = 3
    block[204] = 2
    block[0] = 0x21
    block[128] = 0x03
    block[64] = 0x21
    block[160] = 0x01
    x = np.zeros(256, np.float32)
    x[0], x[16], x[64], x[128], x[192] = 1, -1, 2, -2, 4
    assert O.q6_k_matvec_ref(block, 1, 256, x)[0] == -315.0
    assert O.q6_k_matvec_f64(block, 1, 256, x)[0] == -315.0
    assert O.q6_k_matvec_f32(block, 1, 256, x)[0] == -315.0


def test_q6_k_hand_block_rust():
    block = np.zeros(210, np.uint8)
    block[0:128] = 0x55
    for i in range(16):
        block[192 + i] = (i - 8) & 0xFF
    block[208:210] = [0x00, 0x3C]
    out = O.q6_k_dequant_block_f64(block)
    for e in range(256):
        assert out[e] == (e // 16 - 8) * -27.0
    block[128:192] = 0b11100100
    q = O.q6_k_unpack(block)
    assert q[0] == 5 - 32 and q[32] == 5 + 16 - 32 and q[64] == 5 and q[96] == 5 + 48 - 32
    assert q[128 + 64] == 5


def test_q6_k_swift_and_rust_decoders_agree_and_gate():
    # Swift generator (main.swift:1028-1043) for 64 x 512
    r = O.SplitMix64(555)
    out = bytearray()
    for _ in range(64 * 2):
        for _ in range(208):
            out.append(r.next() & 0xFF)
        scale = np.float16(np.float32(r.uniform_swift()) * np.float32(2) - np.float32(1))
        bits = int(scale.view(np.uint16))
        out += bytes([bits & 0xFF, bits >> 8])
    w = np.frombuffer(bytes(out), np.uint8)
    x = O.seeded_input_swift(512, 202)
    for b in range(0, w.size, 210):
        swift = O.q6_k_decode_block(w[b:b + 210])
        rust = O.q6_k_dequant_block_f32(w[b:b + 210])
        assert np.array_equal(swift.view(np.uint32), rust.view(np.uint32))
    ref64 = O.q6_k_matvec_f64(w, 64, 512, x)
    assert O.max_rel_err(O.q6_k_matvec_ref(w, 64, 512, x), ref64) < 1e-4
    # Rust gate: 3 x 512, d = 0.0625 (lib.rs:526-541)
    r = O.SplitMix64(7)
    w2 = np.zeros(3 * 2 * 210, np.uint8)
    for c in range(6):
        for i in range(208):
            w2[c * 210 + i] = r.next() & 0xFF
        w2[c * 210 + 208: c * 210 + 210] = [0x00, 0x2C]
    x2 = np.array([r.signed_unit_rust() for _ in range(512)], np.float32)
    assert O.max_rel_err(O.q6_k_matvec_f32(w2, 3, 512, x2), O.q6_k_matvec_f64(w2, 3, 512, x2)) < 1e-4
    with pytest.raises(O.OracleError):
        O.q6_k_matvec_f32(w2[1:], 3, 512, x2)


def test_q8_quantizer_half_step_bound():
    # rust/crates/lev-cpu/src/lib.rs:542-557
    r = O.SplitMix64(11)
    x = np.array([r.signed_unit_rust() * np.float32(3.0) for _ in range(96)], np.float32)
    q, d, s = O.quantize_q8(x)
    for i, v in enumerate(x):
        assert abs(q[i] * d[i // 32] - v) <= d[i // 32] * 0.5001
    for g in range(3):
        assert abs(s[g] - d[g] * int(q[g * 32:(g + 1) * 32].astype(np.int32).sum())) < 1e-5
    q0, d0, _ = O.quantize_q8(np.zeros(32, np.float32))
    assert not q0.any() and d0[0] == 0.0


# ---- MoE region (Sources/leviathan-tests/main.swift:8925-8965) ----
def _blk(lo, hi, q):
    return [lo, hi] + [q] * 16


def test_moe_region_hand_computed():
    gu = []
    for _ in range(32):
        gu += _blk(0x00, 0x3C, 0x98)
    for _ in range(32):
        gu += _blk(0x00, 0x30, 0x98)
    dn = []
    for _ in range(32):
        dn += _blk(0x00, 0x38, 0x99)
    ones = np.ones(32, np.float32)
    gate, up, act, d = O.moe_region_f64(32, 32, 1, gu, dn, ones)
    assert np.all(gate == 16) and np.all(up == 2) and np.all(act == 32) and np.all(d == 512)
    assert abs(O.gelu_tanh_up(1, 1) - 0.841192) < 1e-6
    assert O.gelu_tanh_up(-20, 3) == 0
    assert abs(O.gelu_tanh_up_f32(1, 1) - 0.841192) < 1e-6
    bad = list(gu)
    bad[1] = 0x7C
    with pytest.raises(O.OracleError) as e:
        O.moe_region_f64(32, 32, 1, bad, dn, ones)
    assert e.value.name == "nonFiniteScale"
    nanx = ones.copy()
    nanx[3] = np.nan
    with pytest.raises(O.OracleError):
        O.moe_region_f64(32, 32, 1, gu, dn, nanx)


# ---- router / grouping / combine: unpinned by the reference; own cases ----
def test_router_topk_order_ties_and_renormalisation():
    scores = np.array([0.5, 2.0, 2.0, -1.0, 1.0, 2.0, 0.0, 0.25], np.float32)
    idx, w = O.router_topk(scores, 4)
    assert idx.tolist() == [1, 2, 5, 4]  # ties go to the lower index
    assert abs(float(w.sum()) - 1.0) < 1e-6
    e = np.exp(scores.astype(np.float64) - 2.0)
    p = e / e.sum()
    ref = (p[[1, 2, 5, 4]] / p[[1, 2, 5, 4]].sum()).astype(np.float32)
    assert np.array_equal(w, ref)
    idx2, w2 = O.router_topk(scores, 2, expert_scale=np.arange(8, dtype=np.float32))
    assert idx2.tolist() == [1, 2] and w2[0] == np.float32(0.5) * 1 and w2[1] == np.float32(0.5) * 2
    with pytest.raises(O.OracleError):
        O.router_topk(np.array([1.0, np.inf], np.float32), 1)


def test_router_logits_order_is_the_documented_one():
    rng = np.random.default_rng(3)
    w = rng.standard_normal((5, 96)).astype(np.float32)
    x = rng.standard_normal(96).astype(np.float32)
    got = O.router_logits(w, x)
    for e in range(5):
        p = [0.0] * 32
        for l in range(32):
            acc = 0.0
            for i in range(l, 96, 32):
                acc = math.fma(float(w[e, i]), float(x[i]), acc) if hasattr(math, "fma") else acc + float(w[e, i]) * float(x[i])
            p[l] = acc
        for dist in (16, 8, 4, 2, 1):
            p = [p[l] + p[l ^ dist] for l in range(32)]
        if hasattr(math, "fma"):
            assert got[e] == np.float32(p[0])
        else:
            assert abs(got[e] - p[0]) < 1e-5


def test_grouping_is_a_stable_counting_sort():
    idx = np.array([[3, 1], [1, 0], [3, 2], [1, 3]], np.int32)
    counts, offsets, perm = O.group_tokens(idx, 5)
    assert counts.tolist() == [1, 3, 1, 3, 0]
    assert offsets.tolist() == [0, 1, 4, 5, 8, 8]
    assert perm.tolist() == [3, 1, 2, 6, 5, 0, 4, 7]


def test_combine_is_rank_ordered_f32_axpy():
    y = np.array([[1e8, 1.0], [-1e8, 1.0], [1.0, 1.0]], np.float32)
    w = np.array([1.0, 1.0, 0.5], np.float32)
    out = O.combine(y, w)
    assert out.tolist() == [0.5, 2.5]


def test_rmsnorm_known_answers():
    # rust/crates/lev-model/src/lib.rs:432-435: a constant vector normalises to its weight
    for fn in (O.rmsnorm_f32, O.rmsnorm_f64):
        y = fn(np.full(8, 2.0, np.float32), np.full(8, 0.5, np.float32), 1e-6)
        assert np.all(np.abs(y - 0.5) < 1e-5)
    # the definition: x * (1 / sqrt(mean(x^2) + eps)) * w, and no scale without a weight
    x = np.array([[3.0, -4.0, 0.0, 0.0], [1.0, 1.0, 1.0, 1.0]], np.float32)
    w = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    inv0 = 1.0 / np.sqrt(25.0 / 4.0 + 1e-6)
    np.testing.assert_allclose(O.rmsnorm_f64(x, w, 1e-6)[0], np.array([3.0, -8.0, 0.0, 0.0]) * inv0, rtol=1e-12)
    np.testing.assert_allclose(O.rmsnorm_f64(x, None, 1e-6)[1], np.full(4, 1.0 / np.sqrt(1.0 + 1e-6)), rtol=1e-7)
    # the serial f32 form is itself measured against the f64 one, not assumed exact
    big = Q.normal(9, (3, 2816), 1.0).astype(np.float32)
    wb = (1.0 + Q.normal(10, (2816,), 0.1)).astype(np.float32)
    assert O.max_rel_err(O.rmsnorm_f32(big, wb).reshape(-1), O.rmsnorm_f64(big, wb).reshape(-1)) < 1e-5
    # epsilon keeps the zero vector finite
    assert np.all(O.rmsnorm_f32(np.zeros(16, np.float32), None, 1e-6) == 0.0)


def test_attention_oracle_analytic_cases():
    """The reference holds no known-answer vector for attention (its f64 oracle,
    AttentionLowering.swift:358-388, is only compared with its kernels), so the restatement is held to
    cases with closed forms."""
    rng = np.random.default_rng(3)
    hd, kvh, qh, T = 8, 2, 4, 6
    q = rng.standard_normal((qh, hd)).astype(np.float32)
    v = rng.standard_normal((T, kvh, hd)).astype(np.float32)
    # equal keys: plain mean of V of the head's KV head (query heads 0,1 -> KV head 0; 2,3 -> 1)
    k = np.ones((T, kvh, hd), np.float32)
    out = O.attention_f64(q, k, v)
    for h in range(qh):
        np.testing.assert_allclose(out[h], v[:, h // 2].astype(np.float64).mean(axis=0), rtol=1e-12)
    # one position: its V row exactly
    np.testing.assert_array_equal(O.attention_f64(q, k[:1], v[:1])[3], v[0, 1].astype(np.float64))
    # a window of 2 sees the last two positions only
    np.testing.assert_allclose(O.attention_f64(q, k, v, window=2)[0], v[-2:, 0].astype(np.float64).mean(axis=0), rtol=1e-12)
    # a key aligned with the query and far larger takes all the weight; scale 0 removes the preference
    k2 = np.zeros((T, kvh, hd), np.float32)
    k2[4, 0] = 100.0 * q[0] / np.dot(q[0], q[0])
    np.testing.assert_allclose(O.attention_f64(q, k2, v)[0], v[4, 0], rtol=1e-9, atol=1e-30)
    np.testing.assert_allclose(O.attention_f64(q, k2, v, scale=0.0)[0], v[:, 0].astype(np.float64).mean(axis=0), rtol=1e-12)
    # two positions, scores 0 and ln 3: weights 1/4 and 3/4
    k3 = np.zeros((2, 1, hd), np.float32)
    q3 = np.zeros((1, hd), np.float32)
    q3[0, 0], k3[1, 0, 0] = 1.0, np.float32(np.log(3.0))
    v3 = np.stack([np.full((1, hd), 4.0, np.float32), np.full((1, hd), 8.0, np.float32)])
    np.testing.assert_allclose(O.attention_f64(q3, k3, v3)[0], np.full(hd, 7.0), rtol=1e-6)


def test_head_norm_rope_oracle_closed_forms():
    hd = 8
    x = np.zeros((2, hd), np.float32)
    x[0, 0] = 2.0           # norm: 2 / sqrt(4/8) = 2 sqrt 2 at element 0
    x[1, :] = 1.0
    inv = np.array([np.pi / 2, 0.0, 0.0, 0.0], np.float32)  # pair (0, 4) turns by pos * 90 degrees
    out = O.head_norm_rope_f64(x, None, 0.0, inv, 1)
    np.testing.assert_allclose(out[0], [0, 0, 0, 0, 2 * np.sqrt(2), 0, 0, 0], atol=1e-6)   # (a, 0) -> (0, a)
    np.testing.assert_allclose(out[1], [-1, 1, 1, 1, 1, 1, 1, 1], atol=1e-6)               # (1, 1) -> (-1, 1)
    np.testing.assert_allclose(O.head_norm_rope_f64(x, None, 0.0, inv, 0)[1], np.ones(hd), atol=1e-12)  # position 0: no turn
    np.testing.assert_allclose(O.head_norm_rope_f64(x, None, 0.0, None, 7), O.rmsnorm_f64(x, None, 0.0), rtol=1e-12)
    # a turn keeps each pair's length
    r = np.random.default_rng(1).standard_normal((3, hd)).astype(np.float32)
    a = O.head_norm_rope_f64(r, None, 1e-6, np.array([0.3, 0.02, 1.7, 0.9], np.float32), 123)
    b = O.rmsnorm_f64(r, None, 1e-6)
    np.testing.assert_allclose(a[:, :4] ** 2 + a[:, 4:] ** 2, b[:, :4] ** 2 + b[:, 4:] ** 2, rtol=1e-9)
