"""Prefill dequant-GEMM against the rounded-operand f64 oracle
(rust/crates/lev-cli/src/main.rs:1201-1275), through the C ABI."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

# north-star pass bar for bf16 tensor-core prefill, and the reference's own f16 gate
PASS_TOL, REPORT_TOL = 2e-2, 1e-3


@pytest.fixture(scope="module")
def ctx():
    c = lev.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("name,rows,cols,tokens", [
    ("q4_k", 256, 1024, 64), ("q4_k", 80, 512, 37), ("q6_k", 128, 768, 70), ("q4_0", 96, 704, 5), ("q4_0", 64, 2816, 128),
    # several row tiles with a ragged last one, two token tiles (256 + 44)
    ("q4_k", 400, 512, 300), ("q6_k", 360, 256, 130),
    # decode batches against tensors of a few row tiles: raw bytes staged in shared memory, K split over the grid
    # (11 groups of 256 columns over 8 splits; 8 groups over 8; a ragged last row tile; one token)
    ("q4_0", 528, 2816, 32), ("q4_k", 352, 2048, 32), ("q4_k", 200, 1024, 128), ("q4_0", 176, 512, 1),
])
def test_gemm_matches_rounded_operand_oracle(ctx, name, rows, cols, tokens):
    t = H.TYPES[name]
    w = H.quantized(t, 21, rows, cols)
    x = Q.normal(22, (tokens, cols), 1.0)
    wh = ctx.upload(w, t, rows, cols)
    xb = ctx.act_bf16(torch.from_numpy(x).cuda())
    # the conversion is round-to-nearest-even like torch's
    assert torch.equal(xb, torch.from_numpy(x).cuda().to(torch.bfloat16))
    buf, view = H.guarded(tokens * rows)
    y = ctx.gemm_prefill(wh, xb, out=view.view(tokens, rows))
    torch.cuda.synchronize()
    assert H.guards_intact(buf, tokens * rows)
    y = y.cpu().numpy()
    step = 13 if rows > 64 else 1  # every 13th row x all tokens, like the reference's gate
    ref = O.gemm_rounded_f64(t, w, rows, cols, x, "bf16", 0, step)
    err = O.max_rel_err(y[:, ::step], ref)
    assert err < REPORT_TOL and err < PASS_TOL, (name, err)
    y2 = ctx.gemm_prefill(wh, xb).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))
    wh.free()


def test_gemm_rejections(ctx):
    w = H.quantized(Q.GGML_Q4_K, 1, 64, 256)
    wh = ctx.upload(w, Q.GGML_Q4_K, 64, 256)
    with pytest.raises(lev.LevError) as e:
        ctx.lib.lev_gemm_prefill.restype  # keep the binding imported
        ctx._check(ctx.lib.lev_gemm_prefill(ctx.handle, wh.handle, 1, 0, 1, 0))
    assert e.value.name == "badDimensions"
    wh.free()
