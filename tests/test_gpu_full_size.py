"""Full-size checks (the bench's shapes).  The f64 oracle is applied to row samples; whole-tensor
agreement is checked through properties that do not need it: two independent GPU schedules
(bit-exact-decode plain kernel, tensor-core stream kernel) against each other, a matvec as the
concatenation of its row windows, and linearity in the activations."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

FULL = [("q4_k", 12288, 4096), ("q6_k", 4096, 12288), ("q4_0", 4096, 4096)]


@pytest.fixture(scope="module")
def ctx():
    c = lev.Context(0)
    yield c
    c.close()


def _tensor(t, rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn((rows, cols), generator=g, device="cuda") * 0.02
    return Q.quantize(t, w)


def _rel(a, b):
    return float(np.max(np.abs(a - b) / np.maximum(1.0, np.abs(b))))


@pytest.mark.parametrize("name,rows,cols", FULL)
def test_full_size_matvec_properties(ctx, name, rows, cols):
    t = H.TYPES[name]
    wq = _tensor(t, rows, cols, 31)
    wh = ctx.upload(wq, t, rows, cols)
    g = torch.Generator(device="cuda").manual_seed(32)
    x1 = torch.randn((1, cols), generator=g, device="cuda")
    x2 = torch.randn((1, cols), generator=g, device="cuda")
    ys = ctx.matvec(wh, x1, schedule=lev.SCHEDULE_STREAM).cpu().numpy()[0]
    yp = ctx.matvec(wh, x1, schedule=lev.SCHEDULE_PLAIN).cpu().numpy()[0]
    # two independent schedules agree over every row
    assert _rel(ys, yp.astype(np.float64)) < 1e-4
    # sampled rows against the f64 oracle
    bpr = {"q4_k": (cols // 256) * 144, "q6_k": (cols // 256) * 210, "q4_0": (cols // 32) * 18}[name]
    wb = wq.cpu().numpy()
    x1h = x1.cpu().numpy()[0]
    for r0 in (0, rows // 2 + 5, rows - 3):
        ref = O.matvec_f64(t, wb[r0 * bpr:(r0 + 3) * bpr], 3, cols, x1h)
        assert _rel(ys[r0:r0 + 3], ref) < H.REPORT_TOL
    # a matvec is the concatenation of its (16-aligned) row windows
    cut = (rows // 3) // 16 * 16
    a = ctx.matvec(wh, x1, row0=0, rows=cut, schedule=lev.SCHEDULE_STREAM).cpu().numpy()[0]
    b = ctx.matvec(wh, x1, row0=cut, rows=rows - cut, schedule=lev.SCHEDULE_STREAM).cpu().numpy()[0]
    assert _rel(np.concatenate([a, b]), ys.astype(np.float64)) < 1e-5
    # linearity: W(x1 + 2 x2) = W x1 + 2 W x2 (to f32 rounding of the inputs and sums)
    y2 = ctx.matvec(wh, x2, schedule=lev.SCHEDULE_STREAM).cpu().numpy()[0]
    y12 = ctx.matvec(wh, x1 + 2.0 * x2, schedule=lev.SCHEDULE_STREAM).cpu().numpy()[0]
    assert _rel(y12, ys.astype(np.float64) + 2.0 * y2.astype(np.float64)) < 1e-4
    # n = 2 columns give each column's own result
    yy = ctx.matvec(wh, torch.cat([x1, x2]), schedule=lev.SCHEDULE_STREAM).cpu().numpy()
    assert _rel(yy[0], ys.astype(np.float64)) < 1e-5 and _rel(yy[1], y2.astype(np.float64)) < 1e-5
    # n = 4 and n = 8 columns: sampled rows of every column against the f64 oracle, and the first two
    # columns against their single-column results over every row
    x8 = torch.cat([x1, x2, torch.randn((6, cols), generator=g, device="cuda")])
    x8h = x8.cpu().numpy()
    for n in (4, 8):
        yn = ctx.matvec(wh, x8[:n].contiguous(), schedule=lev.SCHEDULE_STREAM).cpu().numpy()
        assert _rel(yn[0], ys.astype(np.float64)) < 1e-5 and _rel(yn[1], y2.astype(np.float64)) < 1e-5
        for r0 in (16, rows // 2 + 5, rows - 3):
            for c in range(n):
                ref = O.matvec_f64(t, wb[r0 * bpr:(r0 + 3) * bpr], 3, cols, x8h[c])
                assert _rel(yn[c, r0:r0 + 3], ref) < H.REPORT_TOL, (name, n, c, r0)
    wh.free()


@pytest.mark.parametrize("name,rows,cols", FULL)
def test_full_size_dequantize_checksum(ctx, name, rows, cols):
    """Bit-exact block decode at full size: sampled rows equal the oracle's, and the whole tensor's
    bit pattern checksum equals the checksum of row-window decodes."""
    t = H.TYPES[name]
    wq = _tensor(t, rows, cols, 41)
    wh = ctx.upload(wq, t, rows, cols)
    full = np.asarray(ctx.dequantize(wh))
    bpr = wq.numel() // rows
    wb = wq.cpu().numpy()
    for r0 in (0, rows // 2, rows - 2):
        ref = O.dequantize_rows(t, wb[r0 * bpr:(r0 + 2) * bpr], 2, cols)
        assert np.array_equal(full[r0:r0 + 2].view(np.uint32), ref.view(np.uint32))
    whole = int(full.view(np.uint32).astype(np.uint64).sum())
    half = rows // 2
    parts = int(np.asarray(ctx.dequantize(wh, 0, half)).view(np.uint32).astype(np.uint64).sum()) + \
        int(np.asarray(ctx.dequantize(wh, half, rows - half)).view(np.uint32).astype(np.uint64).sum())
    assert whole == parts
    wh.free()


def test_full_size_prefill_gemm_samples(ctx):
    """cfg3: X bf16 [512 x 4096] x Q4_K [12288 x 4096]; every 997th row against the rounded-operand
    f64 oracle, all tokens."""
    rows, cols, tokens = 12288, 4096, 512
    t = H.TYPES["q4_k"]
    wq = _tensor(t, rows, cols, 51)
    wh = ctx.upload(wq, t, rows, cols)
    x = Q.normal(52, (tokens, cols), 1.0)
    xb = ctx.act_bf16(torch.from_numpy(x).cuda())
    y = ctx.gemm_prefill(wh, xb).cpu().numpy()
    ref = O.gemm_rounded_f64(t, wq.cpu().numpy(), rows, cols, x, "bf16", 0, 997)
    err = O.max_rel_err(y[:, ::997], ref)
    assert err < 1e-3, err
    wh.free()
