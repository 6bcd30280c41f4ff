"""ctypes binding of the CPU oracle (liblev_oracle.so).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the product package never does.  Every wrapper takes and returns
numpy arrays and raises OracleError on a non-zero status, mirroring the
typed errors of the reference (Sources/LeviathanCore/Q4.swift:17-31,
rust/crates/lev-cpu/src/lib.rs:76-81).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

GGML_Q4_0, GGML_Q4_K, GGML_Q6_K = 2, 12, 14
BLOCK = {GGML_Q4_0: (32, 18), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}

STATUS_NAMES = {
    1: "badDimensions",
    2: "wrongInputCount",
    3: "nonFiniteInput",
    4: "nonFiniteScale",
    5: "nonFiniteOutput",
}


class OracleError(Exception):
    def __init__(self, status: int):
        super().__init__(STATUS_NAMES.get(status, f"status {status}"))
        self.status = status
        self.name = STATUS_NAMES.get(status, str(status))


def build(native_out: str | None = None) -> str:
    """Compile the oracle; with native_out also a -march=native copy there."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    if native_out:
        os.makedirs(native_out, exist_ok=True)
        subprocess.run(["make", "-C", _HERE, "-s", "native", f"OUT={native_out}"], check=True)
        return os.path.join(native_out, "liblev_oracle_native.so")
    return os.path.join(_HERE, "liblev_oracle.so")


def _load(path: str | None = None) -> C.CDLL:
    path = path or os.path.join(_HERE, "liblev_oracle.so")
    if not os.path.exists(path):
        build()
    lib = C.CDLL(path)
    u8p, f32p, f64p, i32p, i8p = (C.c_void_p,) * 5
    L, Z = C.c_long, C.c_size_t

    def sig(name, res, *args):
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("lev_or_f16_to_f64", C.c_double, C.c_uint16)
    sig("lev_or_f16_to_f32", C.c_float, C.c_uint16)
    sig("lev_or_f32_to_f16_bits", C.c_uint16, C.c_float)
    sig("lev_or_f32_to_bf16_bits", C.c_uint16, C.c_float)
    sig("lev_or_bf16_to_f32", C.c_float, C.c_uint16)
    sig("lev_or_splitmix_next", C.c_uint64, C.POINTER(C.c_uint64))
    sig("lev_or_splitmix_uniform_swift", C.c_float, C.POINTER(C.c_uint64))
    sig("lev_or_splitmix_signed_unit_rust", C.c_float, C.POINTER(C.c_uint64))
    sig("lev_or_q4_0_decode_block", C.c_int, u8p, f32p)
    for n in ("lev_or_q4_0_matvec_f32", "lev_or_q4_0_matvec_f64", "lev_or_q4_0_matvec_f32_interleaved",
              "lev_or_q4_k_matvec_f32", "lev_or_q4_k_matvec_f64", "lev_or_q6_k_matvec_ref",
              "lev_or_q6_k_matvec_f64", "lev_or_q6_k_matvec_f32"):
        sig(n, C.c_int, u8p, Z, L, L, f32p, L, C.c_void_p)
    sig("lev_or_q4_0_matvec_f64_dx", C.c_int, u8p, Z, Z, L, L, f64p, L, f64p)
    sig("lev_or_q4_k_unpack_scale_min", None, C.c_int, u8p, u8p, u8p)
    sig("lev_or_q4_k_pack_scale_min", None, u8p, u8p, u8p)
    sig("lev_or_q4_k_dequant_block_f32", None, u8p, f32p)
    sig("lev_or_q4_k_dequant_block_f64", None, u8p, f64p)
    sig("lev_or_q6_k_decode_block", C.c_int, u8p, f32p)
    sig("lev_or_q6_k_unpack", None, u8p, i8p)
    sig("lev_or_q6_k_dequant_block_f32", None, u8p, f32p)
    sig("lev_or_q6_k_dequant_block_f64", None, u8p, f64p)
    sig("lev_or_max_rel_err", C.c_double, f32p, L, f64p, L)
    sig("lev_or_quantize_q8", None, f32p, L, i8p, f32p, f32p)
    sig("lev_or_rmsnorm_f32", None, f32p, L, L, f32p, C.c_float, f32p)
    sig("lev_or_rmsnorm_f64", None, f32p, L, L, f32p, C.c_float, f64p)
    sig("lev_or_head_norm_rope_f64", None, f32p, L, L, f32p, C.c_float, f32p, L, f64p)
    sig("lev_or_attention_f64", C.c_int, f32p, f32p, f32p, L, L, L, L, L, C.c_double, f64p)
    sig("lev_or_gelu_tanh_up", C.c_double, C.c_double, C.c_double)
    sig("lev_or_gelu_tanh_up_f32", C.c_float, C.c_float, C.c_float)
    sig("lev_or_moe_region_f64", C.c_int, L, L, L, u8p, Z, u8p, Z, f32p, f64p, f64p, f64p, f64p)
    sig("lev_or_router_logits", None, f32p, L, L, f32p, f32p)
    sig("lev_or_router_topk", C.c_int, f32p, L, L, f32p, i32p, f32p)
    sig("lev_or_group_tokens", None, i32p, L, L, L, i32p, i32p, i32p)
    sig("lev_or_combine", None, f32p, f32p, L, L, f32p)
    sig("lev_or_moe_token", C.c_int, L, L, L, L, f32p, u8p, u8p, f32p, i32p, f32p, f32p, f64p)
    sig("lev_or_gemm_rounded_f64", C.c_int, C.c_int, u8p, L, L, f32p, L, C.c_int, L, L, f64p)
    sig("lev_or_dequantize_rows", C.c_int, C.c_int, u8p, L, L, f32p)
    sig("lev_or_matvec_threaded", C.c_int, C.c_int, u8p, Z, L, L, f32p, f32p, C.c_int)
    sig("lev_or_hardware_threads", C.c_int)
    return lib


_lib = None


def lib(path: str | None = None) -> C.CDLL:
    global _lib
    if path is not None:
        return _load(path)
    if _lib is None:
        _lib = _load()
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(bytes(a), dtype=np.uint8) if isinstance(a, (bytes, bytearray, list)) else a, dtype=np.uint8)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _check(st: int):
    if st != 0:
        raise OracleError(st)


# ---- conversions ----
def f16_to_f64(h: int) -> float:
    return lib().lev_or_f16_to_f64(h)


def f16_to_f32(h: int) -> float:
    return lib().lev_or_f16_to_f32(h)


def f32_to_f16_bits(v: float) -> int:
    return lib().lev_or_f32_to_f16_bits(v)


def f32_to_bf16_bits(v: float) -> int:
    return lib().lev_or_f32_to_bf16_bits(v)


# ---- generators ----
class SplitMix64:
    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def next(self) -> int:
        return lib().lev_or_splitmix_next(C.byref(self.state))

    def uniform_swift(self) -> float:
        return lib().lev_or_splitmix_uniform_swift(C.byref(self.state))

    def signed_unit_rust(self) -> float:
        return lib().lev_or_splitmix_signed_unit_rust(C.byref(self.state))


def seeded_input_swift(dim: int, seed: int) -> np.ndarray:
    """seededInput of Sources/leviathan-tests/main.swift:65-68."""
    r = SplitMix64(seed)
    return np.array([r.uniform_swift() for _ in range(dim)], dtype=np.float32)


# ---- Q4_0 ----
def q4_0_decode_block(block) -> np.ndarray:
    b = _u8(block)
    if b.size != 18:
        raise OracleError(1)
    out = np.empty(32, np.float32)
    _check(lib().lev_or_q4_0_decode_block(_p(b), _p(out)))
    return out


def _matvec(fn, w, out_dim, in_dim, x, dtype):
    w = _u8(w)
    x = _f32(x)
    y = np.empty(out_dim if out_dim > 0 else 0, dtype)
    _check(fn(_p(w), w.size, out_dim, in_dim, _p(x), x.size, _p(y)))
    return y


def q4_0_matvec_f32(w, out_dim, in_dim, x):
    return _matvec(lib().lev_or_q4_0_matvec_f32, w, out_dim, in_dim, x, np.float32)


def q4_0_matvec_f64(w, out_dim, in_dim, x):
    return _matvec(lib().lev_or_q4_0_matvec_f64, w, out_dim, in_dim, x, np.float64)


def q4_0_matvec_f32_interleaved(w, out_dim, in_dim, x):
    return _matvec(lib().lev_or_q4_0_matvec_f32_interleaved, w, out_dim, in_dim, x, np.float32)


def q4_0_matvec_f64_dx(w, byte_offset, out_dim, in_dim, x):
    w = _u8(w)
    x = np.ascontiguousarray(x, np.float64)
    y = np.empty(out_dim, np.float64)
    _check(lib().lev_or_q4_0_matvec_f64_dx(_p(w), w.size, byte_offset, out_dim, in_dim, _p(x), x.size, _p(y)))
    return y


# ---- Q4_K ----
def q4_k_unpack_scale_min(j: int, scales12) -> tuple[int, int]:
    s = _u8(scales12)
    sc = np.zeros(1, np.uint8)
    mn = np.zeros(1, np.uint8)
    lib().lev_or_q4_k_unpack_scale_min(j, _p(s), _p(sc), _p(mn))
    return int(sc[0]), int(mn[0])


def q4_k_pack_scale_min(sc8, mn8) -> np.ndarray:
    out = np.zeros(12, np.uint8)
    sc, mn = _u8(sc8), _u8(mn8)
    lib().lev_or_q4_k_pack_scale_min(_p(sc), _p(mn), _p(out))
    return out


def q4_k_dequant_block_f32(block) -> np.ndarray:
    b = _u8(block)
    out = np.empty(256, np.float32)
    lib().lev_or_q4_k_dequant_block_f32(_p(b), _p(out))
    return out


def q4_k_dequant_block_f64(block) -> np.ndarray:
    b = _u8(block)
    out = np.empty(256, np.float64)
    lib().lev_or_q4_k_dequant_block_f64(_p(b), _p(out))
    return out


def q4_k_matvec_f32(w, rows, cols, x):
    return _matvec(lib().lev_or_q4_k_matvec_f32, w, rows, cols, x, np.float32)


def q4_k_matvec_f64(w, rows, cols, x):
    return _matvec(lib().lev_or_q4_k_matvec_f64, w, rows, cols, x, np.float64)


# ---- Q6_K ----
def q6_k_decode_block(block) -> np.ndarray:
    b = _u8(block)
    if b.size != 210:
        raise OracleError(1)
    out = np.empty(256, np.float32)
    _check(lib().lev_or_q6_k_decode_block(_p(b), _p(out)))
    return out


def q6_k_unpack(block) -> np.ndarray:
    b = _u8(block)
    out = np.empty(256, np.int8)
    lib().lev_or_q6_k_unpack(_p(b), _p(out))
    return out


def q6_k_dequant_block_f32(block) -> np.ndarray:
    b = _u8(block)
    out = np.empty(256, np.float32)
    lib().lev_or_q6_k_dequant_block_f32(_p(b), _p(out))
    return out


def q6_k_dequant_block_f64(block) -> np.ndarray:
    b = _u8(block)
    out = np.empty(256, np.float64)
    lib().lev_or_q6_k_dequant_block_f64(_p(b), _p(out))
    return out


def q6_k_matvec_ref(w, out_dim, in_dim, x):
    return _matvec(lib().lev_or_q6_k_matvec_ref, w, out_dim, in_dim, x, np.float32)


def q6_k_matvec_f64(w, out_dim, in_dim, x):
    return _matvec(lib().lev_or_q6_k_matvec_f64, w, out_dim, in_dim, x, np.float64)


def q6_k_matvec_f32(w, rows, cols, x):
    return _matvec(lib().lev_or_q6_k_matvec_f32, w, rows, cols, x, np.float32)


# ---- generic ----
def matvec_f64(ggml_type, w, rows, cols, x):
    return {GGML_Q4_0: q4_0_matvec_f64, GGML_Q4_K: q4_k_matvec_f64, GGML_Q6_K: q6_k_matvec_f64}[ggml_type](w, rows, cols, x)


def matvec_cpu_f32(ggml_type, w, rows, cols, x):
    """The reference's own timed CPU form per type."""
    return {GGML_Q4_0: q4_0_matvec_f32, GGML_Q4_K: q4_k_matvec_f32, GGML_Q6_K: q6_k_matvec_ref}[ggml_type](w, rows, cols, x)


def dequantize_rows(ggml_type, w, rows, cols) -> np.ndarray:
    w = _u8(w)
    out = np.empty((rows, cols), np.float32)
    _check(lib().lev_or_dequantize_rows(ggml_type, _p(w), rows, cols, _p(out)))
    return out


def max_rel_err(got, ref) -> float:
    g = _f32(got).ravel()
    r = np.ascontiguousarray(ref, np.float64).ravel()
    return lib().lev_or_max_rel_err(_p(g), g.size, _p(r), r.size)


def quantize_q8(x):
    x = _f32(x)
    q = np.empty(x.size, np.int8)
    d = np.empty(x.size // 32, np.float32)
    s = np.empty(x.size // 32, np.float32)
    lib().lev_or_quantize_q8(_p(x), x.size, _p(q), _p(d), _p(s))
    return q, d, s


# ---- MoE ----
def rmsnorm_f32(x, w=None, eps: float = 1e-6) -> np.ndarray:
    """[vectors][n] f32, the reference kernel's serial order (Gemma4.swift:4247-4268)."""
    x = np.atleast_2d(_f32(x))
    w = None if w is None else _f32(w)
    y = np.empty_like(x)
    lib().lev_or_rmsnorm_f32(_p(x), x.shape[1], x.shape[0], _p(w), eps, _p(y))
    return y


def rmsnorm_f64(x, w=None, eps: float = 1e-6) -> np.ndarray:
    x = np.atleast_2d(_f32(x))
    w = None if w is None else _f32(w)
    y = np.empty(x.shape, np.float64)
    lib().lev_or_rmsnorm_f64(_p(x), x.shape[1], x.shape[0], _p(w), eps, _p(y))
    return y


def head_norm_rope_f64(x, w=None, eps: float = 1e-6, inv_freq=None, pos: int = 0) -> np.ndarray:
    """x [heads][hd]: RMSNorm per head (weight w or none), then rotary by inv_freq[i] * pos (or none)."""
    x = _f32(x)
    w = None if w is None else _f32(w)
    inv_freq = None if inv_freq is None else _f32(inv_freq)
    out = np.empty(x.shape, np.float64)
    lib().lev_or_head_norm_rope_f64(_p(x), x.shape[0], x.shape[1], _p(w), eps, _p(inv_freq), pos, _p(out))
    return out


def attention_f64(q, k, v, window: int = 0, scale: float = 1.0) -> np.ndarray:
    """q [q_heads][hd], k / v [tokens][kv_heads][hd]; the query is at position tokens - 1
    (AttentionLowering.swift:358-388)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(q.shape, np.float64)
    _check(lib().lev_or_attention_f64(_p(q), _p(k), _p(v), q.shape[0], k.shape[1], q.shape[1], k.shape[0], window, scale, _p(out)))
    return out


def gelu_up_rows(gate_up, inter: int, f64: bool = True) -> np.ndarray:
    """[vectors][2*inter] -> [vectors][inter] through the scalar oracle functions."""
    gu = np.atleast_2d(_f32(gate_up))
    fn = gelu_tanh_up if f64 else gelu_tanh_up_f32
    out = np.empty((gu.shape[0], inter), np.float64 if f64 else np.float32)
    for v in range(gu.shape[0]):
        for e in range(inter):
            out[v, e] = fn(float(gu[v, e]), float(gu[v, inter + e]))
    return out


def gelu_tanh_up(g: float, u: float) -> float:
    return lib().lev_or_gelu_tanh_up(g, u)


def gelu_tanh_up_f32(g: float, u: float) -> float:
    return lib().lev_or_gelu_tanh_up_f32(g, u)


def moe_region_f64(hidden, inter, top_k, gu, dn, x):
    gu, dn, x = _u8(gu), _u8(dn), _f32(x)
    if x.size != hidden:
        raise OracleError(2)
    gate = np.empty((top_k, inter), np.float64)
    up = np.empty((top_k, inter), np.float64)
    act = np.empty((top_k, inter), np.float64)
    dno = np.empty((top_k, hidden), np.float64)
    _check(lib().lev_or_moe_region_f64(hidden, inter, top_k, _p(gu), gu.size, _p(dn), dn.size, _p(x),
                                       _p(gate), _p(up), _p(act), _p(dno)))
    return gate, up, act, dno


def router_logits(router_w, x) -> np.ndarray:
    w = _f32(router_w)
    x = _f32(x)
    experts, hidden = w.shape
    scores = np.empty(experts, np.float32)
    lib().lev_or_router_logits(_p(w), experts, hidden, _p(x), _p(scores))
    return scores


def router_topk(scores, top_k, expert_scale=None):
    s = _f32(scores)
    idx = np.empty(top_k, np.int32)
    wts = np.empty(top_k, np.float32)
    es = None if expert_scale is None else _f32(expert_scale)
    _check(lib().lev_or_router_topk(_p(s), s.size, top_k, _p(es), _p(idx), _p(wts)))
    return idx, wts


def group_tokens(idx, experts):
    idx = np.ascontiguousarray(idx, np.int32)
    tokens, top_k = idx.shape
    counts = np.empty(experts, np.int32)
    offsets = np.empty(experts + 1, np.int32)
    perm = np.empty(tokens * top_k, np.int32)
    lib().lev_or_group_tokens(_p(idx), tokens, top_k, experts, _p(counts), _p(offsets), _p(perm))
    return counts, offsets, perm


def combine(y_slots, weights) -> np.ndarray:
    y = _f32(y_slots)
    w = _f32(weights)
    top_k, hidden = y.shape
    out = np.empty(hidden, np.float32)
    lib().lev_or_combine(_p(y), _p(w), top_k, hidden, _p(out))
    return out


def moe_token(hidden, inter, experts, top_k, router_w, gu_all, dn_all, x):
    rw, gu, dn, x = _f32(router_w), _u8(gu_all), _u8(dn_all), _f32(x)
    idx = np.empty(top_k, np.int32)
    wts = np.empty(top_k, np.float32)
    out = np.empty(hidden, np.float32)
    out64 = np.empty(hidden, np.float64)
    _check(lib().lev_or_moe_token(hidden, inter, experts, top_k, _p(rw), _p(gu), _p(dn), _p(x),
                                  _p(idx), _p(wts), _p(out), _p(out64)))
    return idx, wts, out, out64


def gemm_rounded_f64(ggml_type, w, rows, cols, x, input_type="bf16", r0=0, row_step=13):
    w, x = _u8(w), _f32(x)
    tokens = x.shape[0]
    n = len(range(r0, rows, row_step))
    y = np.empty((tokens, n), np.float64)
    _check(lib().lev_or_gemm_rounded_f64(ggml_type, _p(w), rows, cols, _p(x), tokens,
                                         0 if input_type == "bf16" else 1, r0, row_step, _p(y)))
    return y


def matvec_threaded(ggml_type, w, rows, cols, x, threads, lib_path=None):
    w, x = _u8(w), _f32(x)
    y = np.empty(rows, np.float32)
    _check(lib(lib_path).lev_or_matvec_threaded(ggml_type, _p(w), w.size, rows, cols, _p(x), _p(y), threads))
    return y


def hardware_threads() -> int:
    return lib().lev_or_hardware_threads()


# ---- the ends of a decode step and the step itself ----
def embed_row(ggml_type, w, rows, cols, token: int, scale: float) -> np.ndarray:
    """Row `token` of a quantized tensor times scale: every value decoded as the reference decodes it,
    then one f32 product (g4_q6_embed_row, Sources/LeviathanCore/Gemma4.swift:4210-4245:
    y = d * s * level * scale, left to right in f32; d * s * level is exact in f32)."""
    values, bts = BLOCK[ggml_type]
    row_bytes = cols // values * bts
    one = _u8(w)[token * row_bytes:(token + 1) * row_bytes]
    return (dequantize_rows(ggml_type, one, 1, cols)[0] * np.float32(scale)).astype(np.float32)


def softcap_f64(x, cap: float) -> np.ndarray:
    """cap * tanh(x / cap) (g4_softcap, Gemma4.swift:4496-4503), in f64."""
    return float(cap) * np.tanh(np.asarray(x, np.float64) / float(cap))


def decode_step_f64(cfg, host, token: int, pos: int, k_cache, v_cache) -> dict:
    """One token of one sequence through the synthetic decoder, every product in f64 (stage outputs are
    rounded to f32 where the next oracle function takes f32).  The steps are the subset of
    Gemma4Runner.forwardToken / forwardLayer (Gemma4.swift:3611-3905) the synthetic workload keeps:
    embedding row * sqrt(hidden); per layer RMSNorm -> q, k, v; per-head RMSNorm(q_norm / k_norm / none)
    and rotary on q and k; the new k, v rows (rounded to f16) stored at `pos`; attention over
    [0, pos]; x += Wo a; RMSNorm -> softmax router, top-k, renormalized weights, experts, ordered
    combine; x += that; final RMSNorm -> head -> softcap -> argmax.
    `host[name]` holds GGUF block bytes / f32 arrays by tensor name; k_cache / v_cache are per-layer
    f16 arrays [positions][kv_heads][head_dim] of this sequence, updated in place."""
    H, QH, KVH, HD = cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim
    inv_freq = (cfg.rope_base ** (-np.arange(HD // 2, dtype=np.float64) / (HD // 2))).astype(np.float32)
    x = embed_row(cfg.head_type, host["token_embd"], cfg.vocab, H, token, np.float32(np.sqrt(np.float64(H)))).astype(np.float64)
    routing = []
    for l in range(cfg.layers):
        p = f"blk.{l}."
        h = rmsnorm_f64(x, host[p + "attn_norm"], cfg.eps)[0]
        q = matvec_f64(cfg.weight_type, host[p + "attn_q"], QH * HD, H, h)
        k = matvec_f64(cfg.weight_type, host[p + "attn_k"], KVH * HD, H, h)
        v = matvec_f64(cfg.weight_type, host[p + "attn_v"], KVH * HD, H, h)
        q = head_norm_rope_f64(q.reshape(QH, HD), host[p + "attn_q_norm"], cfg.eps, inv_freq, pos)
        k = head_norm_rope_f64(k.reshape(KVH, HD), host[p + "attn_k_norm"], cfg.eps, inv_freq, pos)
        v = head_norm_rope_f64(v.reshape(KVH, HD), None, cfg.eps, None, pos)
        k_cache[l][pos] = k.astype(np.float16)
        v_cache[l][pos] = v.astype(np.float16)
        a = attention_f64(q, k_cache[l][:pos + 1].astype(np.float32), v_cache[l][:pos + 1].astype(np.float32), 0, cfg.attn_scale)
        x1 = x + matvec_f64(cfg.weight_type, host[p + "attn_output"], H, QH * HD, a.reshape(-1))
        h2 = rmsnorm_f64(x1, host[p + "ffn_norm"], cfg.eps)[0]
        idx, wts, _, out64 = moe_token(H, cfg.expert_inter, cfg.experts, cfg.top_k, host[p + "ffn_gate_inp"],
                                       host[p + "ffn_gate_up_exps"], host[p + "ffn_down_exps"], h2)
        routing.append((idx, wts))
        x = x1 + out64
    hn = rmsnorm_f64(x, host["output_norm"], cfg.eps)[0]
    raw = matvec_f64(cfg.head_type, host["token_embd"], cfg.vocab, H, hn)
    logits = softcap_f64(raw, cfg.softcap)
    return {"x": x, "logits": logits, "token": int(np.argmax(logits)), "routing": routing}
