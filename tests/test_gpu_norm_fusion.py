"""RMSNorm, gelu_tanh(gate) * up and axpy on the GPU, stand-alone and folded into the matvec launch,
against the oracle (f64 statistic; the reference's serial f32 kernel measured beside it)."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = lev.Context(0)
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("vectors,n", [(1, 2816), (1, 4096), (3, 96), (8, 1056), (1, 35), (1, 7), (32, 2816)])
@pytest.mark.parametrize("scaled", [True, False])
def test_rmsnorm_matches_the_oracle(ctx, vectors, n, scaled):
    x = Q.normal(vectors * 1000 + n, (vectors, n), 1.0).astype(np.float32)
    w = (1.0 + Q.normal(n, (n,), 0.1)).astype(np.float32) if scaled else None
    ref = O.rmsnorm_f64(x, w, 1e-6)
    got, inv = ctx.rmsnorm(dev(x), None if w is None else dev(w), 1e-6, want_inverse=True)
    got = got.cpu().numpy()
    assert O.max_rel_err(got.reshape(-1), ref.reshape(-1)) < 1e-6
    assert O.max_rel_err(O.rmsnorm_f32(x, w, 1e-6).reshape(-1), ref.reshape(-1)) < 1e-5  # the serial f32 kernel, for context
    want_inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1) + 1e-6)
    np.testing.assert_allclose(inv.cpu().numpy(), want_inv, rtol=1e-6)
    # repeat-run bit identity, in place, and the cached apply
    again = ctx.rmsnorm(dev(x), None if w is None else dev(w), 1e-6).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    xd = dev(x)
    ctx.rmsnorm(xd, None if w is None else dev(w), 1e-6, out=xd)
    assert np.array_equal(xd.cpu().numpy().view(np.uint32), got.view(np.uint32))
    cached = ctx.rmsnorm_cached(dev(x), inv, None if w is None else dev(w)).cpu().numpy()
    assert np.array_equal(cached.view(np.uint32), got.view(np.uint32))


def test_rmsnorm_known_answer_and_rejections(ctx):
    y = ctx.rmsnorm(dev(np.full(8, 2.0, np.float32)), dev(np.full(8, 0.5, np.float32)), 1e-6).cpu().numpy()
    assert np.all(np.abs(y - 0.5) < 1e-5)
    assert np.all(ctx.rmsnorm(torch.zeros(16, device="cuda"), None, 1e-6).cpu().numpy() == 0.0)
    x = torch.ones((2, 6), device="cuda")
    for bad in (lambda: ctx.rmsnorm(x, None, 1e-6),             # several vectors of a length that is not a multiple of 4
                lambda: ctx.rmsnorm(x[:1], None, -1.0),
                lambda: ctx.rmsnorm(x[:1], None, float("nan"))):
        with pytest.raises(lev.LevError):
            bad()


def test_gelu_up_and_axpy(ctx):
    gu = Q.normal(3, (5, 2 * 704), 2.0).astype(np.float32)
    gu[0, :4] = [60.0, -60.0, 0.0, 1e-8]  # the range where a naive tanh overflows
    got = ctx.gelu_up(dev(gu)).cpu().numpy()
    assert O.max_rel_err(got.reshape(-1), O.gelu_up_rows(gu, 704).reshape(-1)) < 1e-6
    assert np.array_equal(got.view(np.uint32), O.gelu_up_rows(gu, 704, f64=False).view(np.uint32)) or \
        O.max_rel_err(got.reshape(-1), O.gelu_up_rows(gu, 704, f64=False).astype(np.float64).reshape(-1)) < 1e-6
    x, r = Q.normal(4, (1000,), 1.0).astype(np.float32), Q.normal(5, (1000,), 1.0).astype(np.float32)
    want = np.float32(0.75) * x.astype(np.float64) + r
    rd = dev(r)
    assert O.max_rel_err(ctx.axpy(0.75, dev(x), rd).cpu().numpy(), want) < 1e-6
    ctx.axpy(0.75, dev(x), rd, out=rd)  # in place
    assert O.max_rel_err(rd.cpu().numpy(), want) < 1e-6
    with pytest.raises(lev.LevError):
        xd = dev(x)
        ctx.axpy(1.0, xd, rd, out=xd)


FUSED_SHAPES = [("q4_k", 2112, 2816), ("q4_k", 48, 256), ("q6_k", 2816, 2304), ("q6_k", 35, 512), ("q4_0", 2112, 2816),
                ("q4_0", 35, 1056), ("q4_0", 4096, 4096)]


@pytest.mark.parametrize("name,rows,cols", FUSED_SHAPES)
@pytest.mark.parametrize("n_cols", [1, 3, 4, 8])
def test_norm_prologue_matches_norm_then_matvec(ctx, name, rows, cols, n_cols):
    t = H.TYPES[name]
    w = H.quantized(t, 7, rows, cols)
    wh = ctx.upload(w, t, rows, cols)
    x = Q.normal(11, (n_cols, cols), 1.5).astype(np.float32)
    nw = (1.0 + Q.normal(12, (cols,), 0.1)).astype(np.float32)
    fused = ctx.matvec_fused(wh, dev(x), "rmsnorm", dev(nw), 1e-6).cpu().numpy()
    xn = O.rmsnorm_f64(x, nw, 1e-6)
    for c in range(n_cols):
        # the f64 oracle of the composition: f64 norm rounded to f32 as the kernel's activation
        ref = O.matvec_f64(t, w, rows, cols, xn[c].astype(np.float32))
        assert O.max_rel_err(fused[c], ref) < H.REPORT_TOL, (name, rows, cols, c)
    # and against the unfused launches of the same library
    unfused = ctx.matvec(wh, ctx.rmsnorm(dev(x), dev(nw), 1e-6)).cpu().numpy()
    assert O.max_rel_err(fused.reshape(-1), unfused.astype(np.float64).reshape(-1)) < 1e-5
    wh.free()


@pytest.mark.parametrize("name,rows,inter", [("q4_k", 2816, 2304), ("q6_k", 2816, 2304), ("q4_0", 2816, 704), ("q4_0", 35, 96)])
@pytest.mark.parametrize("n_cols", [1, 4, 5])
def test_gelu_prologue_and_residual_epilogue(ctx, name, rows, inter, n_cols):
    t = H.TYPES[name]
    w = H.quantized(t, 8, rows, inter)
    wh = ctx.upload(w, t, rows, inter)
    gu = Q.normal(13, (n_cols, 2 * inter), 1.0).astype(np.float32)
    res = Q.normal(14, (n_cols, rows), 1.0).astype(np.float32)
    act = O.gelu_up_rows(gu, inter, f64=False)
    resd = dev(res)
    got = ctx.matvec_fused(wh, dev(gu), "gelu_up", residual=resd, alpha=0.5).cpu().numpy()
    for c in range(n_cols):
        ref = res[c].astype(np.float64) + 0.5 * O.matvec_f64(t, w, rows, inter, act[c])
        assert O.max_rel_err(got[c], ref) < H.REPORT_TOL, (name, c)
    # accumulate in place: y += W act
    ctx.matvec_fused(wh, dev(gu), "gelu_up", residual=resd, alpha=1.0, out=resd)
    for c in range(n_cols):
        ref = res[c].astype(np.float64) + O.matvec_f64(t, w, rows, inter, act[c])
        assert O.max_rel_err(resd.cpu().numpy()[c], ref) < H.REPORT_TOL
    # no prologue, residual only
    x = Q.normal(15, (n_cols, inter), 1.0).astype(np.float32)
    got = ctx.matvec_fused(wh, dev(x), None, residual=dev(res), alpha=-2.0).cpu().numpy()
    for c in range(n_cols):
        assert O.max_rel_err(got[c], res[c].astype(np.float64) - 2.0 * O.matvec_f64(t, w, rows, inter, x[c])) < H.REPORT_TOL
    wh.free()


@pytest.mark.parametrize("name", ["q4_k", "q4_0"])
@pytest.mark.parametrize("n_cols", [1, 4, 6])
def test_ffn_block_fused_equals_unfused(ctx, name, n_cols):
    """norm -> gate, up -> gelu_up -> down -> residual (Sources/LeviathanCore/Gemma4.swift:3741-3753) in
    two fused launches against six separate ones and against the oracle."""
    t = H.TYPES[name]
    hidden, inter = 2816, 2304 if name == "q4_k" else 2112
    wg, wu = H.quantized(t, 21, inter, hidden), H.quantized(t, 22, inter, hidden)
    td = Q.GGML_Q6_K if name == "q4_k" else t
    wd = H.quantized(td, 23, hidden, inter)
    hg, hu, hd = ctx.upload(wg, t, inter, hidden), ctx.upload(wu, t, inter, hidden), ctx.upload(wd, td, hidden, inter)
    x = Q.normal(24, (n_cols, hidden), 1.0).astype(np.float32)
    nw = (1.0 + Q.normal(25, (hidden,), 0.1)).astype(np.float32)
    xd, nwd = dev(x), dev(nw)
    # fused: gate and up write the halves of one [gate | up] row
    gu = torch.empty((n_cols, 2 * inter), device="cuda")
    if n_cols == 1:
        ctx.matvec_multi_fused([hg, hu], xd, "rmsnorm", nwd, 1e-6, outs=[gu[:, :inter], gu[:, inter:]])
    else:  # rows of the halves are strided for several columns: separate outputs, then one buffer
        g, u = ctx.matvec_multi_fused([hg, hu], xd, "rmsnorm", nwd, 1e-6)
        gu = torch.cat([g, u], dim=1).contiguous()
    out_fused = ctx.matvec_fused(hd, gu, "gelu_up", residual=xd, alpha=1.0).cpu().numpy()
    # unfused
    h = ctx.rmsnorm(xd, nwd, 1e-6)
    g, u = ctx.matvec(hg, h), ctx.matvec(hu, h)
    act = ctx.gelu_up(torch.cat([g.reshape(n_cols, -1), u.reshape(n_cols, -1)], dim=1).contiguous())
    out_unfused = ctx.axpy(1.0, ctx.matvec(hd, act).reshape(n_cols, -1), xd).cpu().numpy()
    assert O.max_rel_err(out_fused.reshape(-1), out_unfused.astype(np.float64).reshape(-1)) < 1e-5
    # oracle of the whole block
    xn = O.rmsnorm_f64(x, nw, 1e-6).astype(np.float32)
    for c in range(n_cols):
        gg = O.matvec_f64(t, wg, inter, hidden, xn[c]).astype(np.float32)
        uu = O.matvec_f64(t, wu, inter, hidden, xn[c]).astype(np.float32)
        a = O.gelu_up_rows(np.concatenate([gg, uu])[None, :], inter, f64=False)[0]
        ref = x[c].astype(np.float64) + O.matvec_f64(td, wd, hidden, inter, a)
        assert O.max_rel_err(out_fused[c], ref) < H.REPORT_TOL, (name, c)
    for h_ in (hg, hu, hd):
        h_.free()


def test_fused_rejections(ctx):
    t = Q.GGML_Q4_0
    wh = ctx.upload(H.quantized(t, 1, 64, 128), t, 64, 128)
    x = torch.ones((1, 128), device="cuda")
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_fused(wh, x, "gelu_up")  # gelu_up expects [gate | up] = 256 values
    assert e.value.name == "wrongInputCount"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_fused(wh, x, "rmsnorm", eps=-1.0)
    assert e.value.name == "badArgument"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_fused(wh, x, None, out=torch.empty(8, device="cuda"))
    assert e.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_fused(wh, x, None, rows=65)
    assert e.value.name == "badDimensions"
    wh.free()


@pytest.mark.parametrize("vectors,n", [(1, 262144), (1, 7), (3, 1000), (32, 4096), (2, 262145), (1, 1)])
def test_argmax_index_and_margin(ctx, vectors, n):
    x = Q.normal(vectors + n, (vectors, n), 1.0).astype(np.float32)
    if n > 8:
        x[0, 5] = x[0, n - 3] = 9.0      # a tie: the lower index wins, the margin is zero
        x[-1, n // 2] = np.nan           # NaN never wins
    idx, margin = ctx.argmax(dev(x), want_margin=True)
    idx, margin = idx.cpu().numpy(), margin.cpu().numpy()
    for v in range(vectors):
        row = np.where(np.isnan(x[v]), -np.inf, x[v])
        want = int(np.argmax(row))
        assert idx[v] == want, (v, idx[v], want)
        if n > 1:
            second = np.partition(row, -2)[-2]
            assert margin[v] == np.float32(row[want] - second)
    if n > 8:
        assert idx[0] == 5 and margin[0] == 0.0
    again = ctx.argmax(dev(x))
    assert np.array_equal(again.cpu().numpy(), idx)


@pytest.mark.parametrize("q_heads,kv_heads,hd,cols", [(16, 8, 256, 1), (4, 2, 128, 3), (8, 0, 64, 2), (2, 2, 512, 1)])
def test_qkv_norm_rope(ctx, q_heads, kv_heads, hd, cols):
    heads = q_heads + 2 * kv_heads
    x = Q.normal(31, (cols, heads * hd), 1.0).astype(np.float32)
    qw = (1.0 + Q.normal(32, (hd,), 0.1)).astype(np.float32)
    kw = (1.0 + Q.normal(33, (hd,), 0.1)).astype(np.float32)
    inv = (10000.0 ** (-np.arange(hd // 2, dtype=np.float64) / (hd // 2))).astype(np.float32)
    pos = np.array([4095, 17, 0][:cols], np.int32)
    xd = dev(x)
    ctx.qkv_norm_rope(xd, q_heads, kv_heads, hd, dev(qw), dev(kw), 1e-6, dev(inv), dev(pos))
    got = xd.cpu().numpy().reshape(cols, heads, hd)
    xr = x.reshape(cols, heads, hd)
    for c in range(cols):
        ref = np.concatenate([
            O.head_norm_rope_f64(xr[c, :q_heads], qw, 1e-6, inv, int(pos[c])),
            O.head_norm_rope_f64(xr[c, q_heads:q_heads + kv_heads], kw, 1e-6, inv, int(pos[c])) if kv_heads else np.empty((0, hd)),
            O.head_norm_rope_f64(xr[c, q_heads + kv_heads:], None, 1e-6, None, 0) if kv_heads else np.empty((0, hd))])
        assert O.max_rel_err(got[c].reshape(-1), ref.reshape(-1)) < 2e-5, (c,)
    # without frequencies: the per-head norms alone, equal to lev_rmsnorm over heads as vectors
    yd = dev(x)
    ctx.qkv_norm_rope(yd, q_heads, kv_heads, hd, None, None, 1e-6, None, None)
    plain = ctx.rmsnorm(dev(x.reshape(cols * heads, hd)), None, 1e-6).cpu().numpy()
    assert O.max_rel_err(yd.cpu().numpy().reshape(-1), plain.astype(np.float64).reshape(-1)) < 1e-6
    with pytest.raises(lev.LevError):
        ctx.qkv_norm_rope(xd, q_heads, kv_heads, hd + 1, None, None, 1e-6, None, None)
    with pytest.raises(lev.LevError):
        ctx.qkv_norm_rope(xd, q_heads, kv_heads, hd, None, None, 1e-6, dev(inv), None)
