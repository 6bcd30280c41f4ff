"""GGUF block encoders and seeded input generators for synthetic workloads.

The reference only decodes GGUF blocks; it has no weight quantizer.  These
encoders are this package's own, written from the block layouts the decoders
define (Sources/LeviathanCore/Q4.swift:33-69, Sources/LeviathanCore/Q6.swift:3-23,
rust/crates/lev-cpu/src/lib.rs:64-130).  They are data preparation, not part
of the measured path, and run on torch tensors of any device.
"""
from __future__ import annotations

import numpy as np
import torch

GGML_Q4_0, GGML_Q4_K, GGML_Q6_K = 2, 12, 14

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, n: int, start: int = 0) -> np.ndarray:
    """n consecutive outputs of SplitMix64(seed) (Sources/LeviathanCore/RNG.swift:11-17),
    beginning with output number `start`; vectorised because output k only
    depends on seed + (k+1)*gamma."""
    with np.errstate(over="ignore"):
        k = np.arange(start + 1, start + n + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + k * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform_swift(seed: int, n: int) -> np.ndarray:
    """nextUniform of Sources/LeviathanCore/RNG.swift:20-23: 53-bit, [-1, 1)."""
    u = (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    return (u.astype(np.float32) * np.float32(2.0) - np.float32(1.0)).astype(np.float32)


def normal(seed: int, shape, sigma: float = 1.0) -> np.ndarray:
    """N(0, sigma) f32 from SplitMix64 by Box-Muller (two outputs per pair of
    53-bit uniforms).  The reference has only a uniform generator; the normal
    transform is this package's choice and is fixed here."""
    n = int(np.prod(shape))
    pairs = (n + 1) // 2
    raw = splitmix64(seed, 2 * pairs)
    u1 = ((raw[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740992.0  # (0, 1]
    u2 = (raw[1::2] >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * pairs, np.float64)
    out[0::2] = r * np.cos(2.0 * np.pi * u2)
    out[1::2] = r * np.sin(2.0 * np.pi * u2)
    return (out[:n] * sigma).astype(np.float32).reshape(shape)


def _wrap_i64(v: int) -> int:
    v &= 0xFFFFFFFFFFFFFFFF
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    """logical shift right of a two's-complement int64 tensor"""
    return (z >> s) & ((1 << (64 - s)) - 1)


def normal_torch(seed: int, shape, sigma: float = 1.0, device="cuda") -> torch.Tensor:
    """The same generator as `normal`, in torch on any device (int64 arithmetic wraps like uint64):
    large synthetic tensors are built on the GPU in milliseconds.  SplitMix64 outputs are identical to
    the bit; the Box-Muller transcendentals run in f64 on the device and are rounded to f32, so a value
    can differ from the numpy form only where the two libraries' f64 results straddle an f32 rounding
    boundary (about one element in 2^29)."""
    n = 1
    for d in shape:
        n *= int(d)
    pairs = (n + 1) // 2
    k = torch.arange(1, 2 * pairs + 1, dtype=torch.int64, device=device)
    z = k * _wrap_i64(0x9E3779B97F4A7C15) + _wrap_i64(seed)
    z = (z ^ _lsr(z, 30)) * _wrap_i64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _wrap_i64(0x94D049BB133111EB)
    z = z ^ _lsr(z, 31)
    del k
    u = _lsr(z, 11).to(torch.float64)
    del z
    u1 = (u[0::2] + 1.0) / 9007199254740992.0
    u2 = u[1::2] / 9007199254740992.0
    del u
    r = torch.sqrt(-2.0 * torch.log(u1))
    ang = 2.0 * np.pi * u2
    out = torch.empty(2 * pairs, dtype=torch.float64, device=device)
    out[0::2] = r * torch.cos(ang)
    out[1::2] = r * torch.sin(ang)
    return (out[:n] * sigma).to(torch.float32).reshape(*shape)


def _f16_bytes(v: torch.Tensor) -> torch.Tensor:
    """f32 tensor [...] -> uint8 [..., 2] little-endian IEEE half bits."""
    return v.to(torch.float16).contiguous().view(torch.uint8).reshape(*v.shape, 2)


def _f16_round(v: torch.Tensor) -> torch.Tensor:
    return v.to(torch.float16).to(torch.float32)


def quantize_q4_0(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> uint8 [rows * cols/32 * 18].  d = (signed value of
    largest magnitude) / -8 stored as fp16; q = trunc(x/d + 8.5) clipped to
    0..15; byte l = q[l] | q[16+l] << 4."""
    rows, cols = w.shape
    assert cols % 32 == 0
    b = w.reshape(rows, cols // 32, 32).to(torch.float32)
    amax_idx = b.abs().argmax(dim=-1, keepdim=True)
    mx = torch.gather(b, -1, amax_idx)
    d = mx / -8.0
    inv = torch.where(d == 0, torch.zeros_like(d), 1.0 / d)
    q = torch.clamp(torch.trunc(b * inv + 8.5), 0, 15).to(torch.uint8)
    qs = q[..., :16] | (q[..., 16:] << 4)
    out = torch.cat([_f16_bytes(d.squeeze(-1)), qs], dim=-1)
    return out.reshape(-1).contiguous()


def _pack_q4_k_scales(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """[..., 8] uint8 scales and mins (0..63) -> [..., 12] packed bytes, the
    layout unpack_scale_min reads (rust/crates/lev-cpu/src/lib.rs:64-74)."""
    s = torch.zeros(*sc.shape[:-1], 12, dtype=torch.uint8, device=sc.device)
    s[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    s[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    return s


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> uint8 [rows * cols/256 * 144].  Per 32-value
    sub-block an affine 4-bit code x ~ d*sc*q - dmin*m with 6-bit sc, m."""
    rows, cols = w.shape
    assert cols % 256 == 0
    b = w.reshape(rows, cols // 256, 8, 32).to(torch.float32)
    lo = torch.clamp(b.amin(dim=-1), max=0.0)
    hi = b.amax(dim=-1)
    scale_f = (hi - lo) / 15.0
    min_f = -lo
    d = _f16_round(scale_f.amax(dim=-1, keepdim=True) / 63.0)
    dmin = _f16_round(min_f.amax(dim=-1, keepdim=True) / 63.0)
    sc = torch.where(d > 0, torch.round(scale_f / torch.where(d > 0, d, torch.ones_like(d))), torch.zeros_like(scale_f))
    mn = torch.where(dmin > 0, torch.round(min_f / torch.where(dmin > 0, dmin, torch.ones_like(dmin))), torch.zeros_like(min_f))
    sc = sc.clamp(0, 63)
    mn = mn.clamp(0, 63)
    step = (d * sc).unsqueeze(-1)
    off = (dmin * mn).unsqueeze(-1)
    q = torch.where(step > 0, torch.round((b + off) / torch.where(step > 0, step, torch.ones_like(step))),
                    torch.zeros_like(b)).clamp(0, 15).to(torch.uint8)
    q = q.reshape(rows, cols // 256, 4, 2, 32)
    qs = (q[:, :, :, 0, :] | (q[:, :, :, 1, :] << 4)).reshape(rows, cols // 256, 128)
    out = torch.cat([_f16_bytes(d.squeeze(-1)), _f16_bytes(dmin.squeeze(-1)),
                     _pack_q4_k_scales(sc.to(torch.uint8), mn.to(torch.uint8)), qs], dim=-1)
    return out.reshape(-1).contiguous()


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> uint8 [rows * cols/256 * 210].  Per 16-value
    sub-block a signed int8 sub-scale; 6-bit levels stored biased by 32."""
    rows, cols = w.shape
    assert cols % 256 == 0
    nb = cols // 256
    b = w.reshape(rows, nb, 16, 16).to(torch.float32)
    amax_idx = b.abs().argmax(dim=-1, keepdim=True)
    mx = torch.gather(b, -1, amax_idx).squeeze(-1)
    scale_f = mx / -32.0
    d = _f16_round(scale_f.abs().amax(dim=-1, keepdim=True) / 127.0)
    sc = torch.where(d > 0, torch.round(scale_f / torch.where(d > 0, d, torch.ones_like(d))), torch.zeros_like(scale_f))
    sc = sc.clamp(-128, 127)
    step = (d * sc).unsqueeze(-1)
    q = torch.where(step != 0, torch.round(b / torch.where(step != 0, step, torch.ones_like(step))),
                    torch.zeros_like(b)).clamp(-32, 31)
    lv = (q + 32).to(torch.uint8).reshape(rows, nb, 2, 4, 32)  # [half c][group of 32][l]
    lo4 = lv & 0x0F
    hi2 = lv >> 4
    ql = torch.empty(rows, nb, 2, 64, dtype=torch.uint8, device=w.device)
    ql[..., 0:32] = lo4[:, :, :, 0, :] | (lo4[:, :, :, 2, :] << 4)
    ql[..., 32:64] = lo4[:, :, :, 1, :] | (lo4[:, :, :, 3, :] << 4)
    qh = hi2[:, :, :, 0, :] | (hi2[:, :, :, 1, :] << 2) | (hi2[:, :, :, 2, :] << 4) | (hi2[:, :, :, 3, :] << 6)
    scb = sc.to(torch.int8).view(torch.uint8)
    out = torch.cat([ql.reshape(rows, nb, 128), qh.reshape(rows, nb, 64), scb, _f16_bytes(d.squeeze(-1))], dim=-1)
    return out.reshape(-1).contiguous()


def quantize(ggml_type: int, w: torch.Tensor) -> torch.Tensor:
    return {GGML_Q4_0: quantize_q4_0, GGML_Q4_K: quantize_q4_k, GGML_Q6_K: quantize_q6_k}[ggml_type](w)


def quantized_normal(ggml_type: int, seed: int, rows: int, cols: int, sigma: float = 0.02,
                     device: str = "cpu") -> torch.Tensor:
    """Seeded N(0, sigma) weights [rows, cols], encoded; uint8 tensor on `device`."""
    w = torch.from_numpy(normal(seed, (rows, cols), sigma)).to(device)
    return quantize(ggml_type, w)


def adversarial_activations(kind: str, n: int) -> np.ndarray:
    """The reference's accuracy-run inputs
    (tools/q4_simd_qualification/main.swift:145-156): a signed sinusoid,
    +-1e-3 alternating, and a one-hot near the last column."""
    i = np.arange(n, dtype=np.float64)
    if kind == "sinusoid":
        return (np.sin(i * 0.137 + 0.31) * (0.5 + 0.5 * np.cos(i * 0.011))).astype(np.float32)
    if kind == "alternating":
        return (np.where(i % 2 == 0, 1.0, -1.0).astype(np.float32) * np.float32(1e-3)).astype(np.float32)
    if kind == "onehot":
        x = np.zeros(n, np.float32)
        x[n - 1] = 0.75
        return x
    raise ValueError(kind)
