"""The package's own GGUF encoders against the oracle decoders and, where it
is installed, against gguf-py as an independent third party."""
import numpy as np
import pytest
import torch

from leviathan_b200 import quant as Q
from oracle import oracle as O


def test_splitmix_vectorised_matches_the_sequential_stream():
    r = O.SplitMix64(0x4C455649)
    seq = np.array([r.next() for _ in range(64)], np.uint64)
    assert np.array_equal(Q.splitmix64(0x4C455649, 64), seq)
    assert np.array_equal(Q.splitmix64(0x4C455649, 10, start=20), seq[20:30])
    assert np.array_equal(Q.uniform_swift(7, 32), O.seeded_input_swift(32, 7))


def test_normal_generator_moments():
    v = Q.normal(3, (200000,), 0.02)
    assert abs(v.mean()) < 2e-4 and abs(v.std() - 0.02) < 2e-4
    assert np.array_equal(v, Q.normal(3, (200000,), 0.02))


@pytest.mark.parametrize("t,tol", [(Q.GGML_Q4_0, 0.0026), (Q.GGML_Q4_K, 0.0040), (Q.GGML_Q6_K, 0.0008)])
def test_encode_decode_round_trip_error(t, tol):
    w = Q.normal(11 + t, (24, 512), 0.02)
    enc = Q.quantize(t, torch.from_numpy(w)).numpy()
    bv, bb = O.BLOCK[t]
    assert enc.size == 24 * 512 // bv * bb
    dec = O.dequantize_rows(t, enc, 24, 512)
    assert np.abs(dec - w).max() < tol * 2.5
    assert np.sqrt(np.mean((dec - w) ** 2)) < tol


def test_q4_0_bytes_equal_gguf_py():
    gguf = pytest.importorskip("gguf")
    w = Q.normal(5, (16, 256), 0.02)
    ours = Q.quantize_q4_0(torch.from_numpy(w)).numpy()
    theirs = gguf.quants.quantize(w, gguf.GGMLQuantizationType.Q4_0).reshape(-1)
    assert np.array_equal(ours, theirs)


@pytest.mark.parametrize("t,name", [(Q.GGML_Q4_0, "Q4_0"), (Q.GGML_Q4_K, "Q4_K"), (Q.GGML_Q6_K, "Q6_K")])
def test_oracle_decode_agrees_with_gguf_py(t, name):
    gguf = pytest.importorskip("gguf")
    w = Q.normal(21 + t, (8, 512), 0.02)
    enc = Q.quantize(t, torch.from_numpy(w)).numpy()
    ours = O.dequantize_rows(t, enc, 8, 512)
    bv, bb = O.BLOCK[t]
    theirs = gguf.quants.dequantize(enc.reshape(8, 512 // bv * bb), getattr(gguf.GGMLQuantizationType, name))
    # gguf-py factors the products differently, so equality is to rounding
    assert np.allclose(ours, theirs.reshape(8, 512), rtol=2e-6, atol=1e-9)


def test_degenerate_blocks_encode_to_zero():
    z = torch.zeros(2, 256)
    for t in (Q.GGML_Q4_0, Q.GGML_Q4_K, Q.GGML_Q6_K):
        dec = O.dequantize_rows(t, Q.quantize(t, z).numpy(), 2, 256)
        assert not dec.any()
