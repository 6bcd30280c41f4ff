"""Shared builders for the GPU parity tests."""
import numpy as np
import torch

from leviathan_b200 import quant as Q
from oracle import oracle as O

TYPES = {"q4_0": Q.GGML_Q4_0, "q4_k": Q.GGML_Q4_K, "q6_k": Q.GGML_Q6_K}
# fp32-path pass bar of the build and the reference's own component gate
PASS_TOL = 1e-3
REPORT_TOL = 1e-4


def quantized(t, seed, rows, cols, sigma=0.02):
    return Q.quantized_normal(t, seed, rows, cols, sigma).numpy()


def random_blocks(t, seed, rows, cols):
    """Uniformly random block bytes with finite, moderate fp16 scales: hits
    saturated quants and mixed-sign sub-scales the encoders rarely produce."""
    bv, bb = O.BLOCK[t]
    n = rows * cols // bv
    raw = (Q.splitmix64(seed, n * bb) & np.uint64(0xFF)).astype(np.uint8).reshape(n, bb)
    halves = np.array([0x2E66, 0x3000, 0x3266, 0x2800, 0x1C00, 0x3400, 0xAE66, 0xB000], np.uint16)
    if t == Q.GGML_Q6_K:
        # int8 sub-scales reach 127 and levels 32: keep d near 2^-9 so that a
        # row's terms stay O(10) and f32 accumulation noise stays below 1e-4
        halves = np.array([0x1400, 0x1800, 0x1C00, 0x1A66, 0x9400, 0x9800, 0x9C00, 0x1666], np.uint16)
    pick = (Q.splitmix64(seed ^ 0x5A5A, 2 * n) % np.uint64(8)).astype(np.int64).reshape(n, 2)
    pos = {Q.GGML_Q4_0: [0], Q.GGML_Q4_K: [0, 2], Q.GGML_Q6_K: [208]}[t]
    for k, p in enumerate(pos):
        h = halves[pick[:, k]]
        if t == Q.GGML_Q4_K:
            h = h & np.uint16(0x7FFF)
        raw[:, p] = (h & np.uint16(0xFF)).astype(np.uint8)
        raw[:, p + 1] = (h >> np.uint16(8)).astype(np.uint8)
    return raw.reshape(-1)


def guarded(n, device="cuda"):
    """NaN-filled output with guard words after it; returns (buffer, view)."""
    buf = torch.full((n + 64,), float("nan"), device=device)
    buf[n:] = 12345.0
    return buf, buf[:n]


def guards_intact(buf, n):
    return bool((buf[n:] == 12345.0).all().item())
