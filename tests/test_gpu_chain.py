"""lev_matvec_chain: a list of one-column products in one launch of the persistent kernel, against
the f64 oracle and against the same steps run one call at a time."""
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


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_independent_ops_of_three_formats_in_one_launch(ctx):
    """Ragged shapes (35 rows, 33 blocks per row, rows below one tile), different activations per op,
    two ops sharing one activation vector; every output against the f64 oracle."""
    specs = [("q4_k", 35, 768, 0), ("q4_k", 96, 768, 0), ("q6_k", 48, 3072, 1), ("q4_0", 35, 33 * 32, 2),
             ("q4_0", 300, 2816, 3), ("q6_k", 9, 256, 4), ("q4_k", 17, 256, 4), ("q4_0", 4096 // 8, 704, 5)]
    xs = {}
    ops, refs, bufs = [], [], []
    handles = []
    for i, (name, rows, cols, xi) in enumerate(specs):
        t = H.TYPES[name]
        key = (xi, cols)
        if key not in xs:
            xs[key] = Q.normal(900 + xi, (cols,), 1.0)
        w = H.quantized(t, 700 + i, rows, cols) if i % 2 == 0 else H.random_blocks(t, 700 + i, rows, cols)
        wh = ctx.upload(w, t, rows, cols)
        handles.append(wh)
        buf, view = H.guarded(rows)
        bufs.append((buf, rows))
        ops.append(dict(w=wh, x=None, out=view, key=key))
        refs.append(O.matvec_f64(t, w, rows, cols, xs[key]))
    xd = {k: _dev(v) for k, v in xs.items()}
    for o in ops:
        o["x"] = xd[o["key"]]
    l0 = ctx.launch_count()
    outs = ctx.matvec_chain(ops)
    assert ctx.launch_count() - l0 == 1
    ctx.synchronize()
    for i, (out, ref) in enumerate(zip(outs, refs)):
        assert H.guards_intact(*bufs[i])
        err = O.max_rel_err(out.cpu().numpy(), ref)
        assert err < (H.REPORT_TOL if i % 2 == 0 else H.PASS_TOL), (specs[i], err)
    # same call, same bits
    first = [o.clone() for o in outs]
    outs2 = ctx.matvec_chain(ops)
    for a, b in zip(first, outs2):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    for h in handles:
        h.free()


@pytest.mark.parametrize("hidden,ffn", [(768, 1024), (4096, 12288)])
def test_dependent_ffn_in_one_launch(ctx, hidden, ffn):
    """norm -> gate, up -> gelu(gate) * up -> down -> residual as three ops of one launch: the third
    waits for the first two on the device.  Against the f64 composition (sampled rows at full size)
    and against the same steps as separate calls."""
    t4, t6 = H.TYPES["q4_k"], H.TYPES["q6_k"]
    if hidden >= 4096:
        g = torch.Generator(device="cuda").manual_seed(5)
        wg = Q.quantize(t4, torch.randn((ffn, hidden), generator=g, device="cuda") * 0.02)
        wu = Q.quantize(t4, torch.randn((ffn, hidden), generator=g, device="cuda") * 0.02)
        wd = Q.quantize(t6, torch.randn((hidden, ffn), generator=g, device="cuda") * 0.02)
    else:
        wg, wu, wd = (_dev(H.quantized(t4, 11, ffn, hidden)), _dev(H.quantized(t4, 12, ffn, hidden)),
                      _dev(H.quantized(t6, 13, hidden, ffn)))
    hg, hu, hd = ctx.upload(wg, t4, ffn, hidden), ctx.upload(wu, t4, ffn, hidden), ctx.upload(wd, t6, hidden, ffn)
    x = _dev(Q.normal(21, (hidden,), 1.0))
    nw = _dev(1.0 + Q.normal(22, (hidden,), 0.02))
    gu = torch.full((2 * ffn,), float("nan"), device="cuda")
    buf, out = H.guarded(hidden)
    ops = [dict(w=hg, x=x, out=gu[:ffn], prologue="rmsnorm", norm_weight=nw, eps=1e-6),
           dict(w=hu, x=x, out=gu[ffn:], prologue="rmsnorm", norm_weight=nw, eps=1e-6),
           dict(w=hd, x=gu, out=out, prologue="gelu_up", residual=x, alpha=1.0)]
    l0 = ctx.launch_count()
    ctx.matvec_chain(ops)
    assert ctx.launch_count() - l0 == 1
    ctx.synchronize()
    assert H.guards_intact(buf, hidden)
    got = out.cpu().numpy()
    # the same steps, one call each
    gu2 = torch.empty_like(gu)
    ctx.matvec_fused(hg, x, prologue="rmsnorm", norm_weight=nw, out=gu2[:ffn].view(1, -1))
    ctx.matvec_fused(hu, x, prologue="rmsnorm", norm_weight=nw, out=gu2[ffn:].view(1, -1))
    sep = ctx.matvec_fused(hd, gu2.view(1, -1), prologue="gelu_up", residual=x.view(1, -1)).cpu().numpy().reshape(-1)
    assert O.max_rel_err(got, sep.astype(np.float64)) < 1e-5
    # f64 composition
    xh, nwh = x.cpu().numpy().astype(np.float64), nw.cpu().numpy().astype(np.float64)
    xn = (xh / np.sqrt(np.mean(xh * xh) + 1e-6) * nwh).astype(np.float32)
    wgb, wub, wdb = wg.cpu().numpy(), wu.cpu().numpy(), wd.cpu().numpy()
    gate = O.matvec_f64(t4, wgb, ffn, hidden, xn)
    up = O.matvec_f64(t4, wub, ffn, hidden, xn)
    act = (0.5 * gate * (1.0 + np.tanh(0.7978845608028654 * (gate + 0.044715 * gate ** 3))) * up).astype(np.float32)
    bpr = (ffn // 256) * 210
    rows = range(hidden) if hidden < 4096 else [0, 1, 17, 2048, 4095]
    for r in rows:
        ref = O.matvec_f64(t6, wdb[r * bpr:(r + 1) * bpr], 1, ffn, act)[0] + xh[r]
        assert abs(got[r] - ref) / max(1.0, abs(ref)) < 2e-4, (r, got[r], ref)
    # repeat runs give the same bits
    out2 = torch.empty_like(out)
    ops[2]["out"] = out2
    ctx.matvec_chain(ops)
    assert torch.equal(out.view(torch.int32), out2.view(torch.int32))
    for h in (hg, hu, hd):
        h.free()


def test_many_small_ops_reuse_table_buffers(ctx):
    """Thirty-two ops with alternating activation vectors: table buffers, records and tickets are
    reused many times inside one launch; shares below one K-step per warp."""
    t = H.TYPES["q4_0"]
    rows, cols = 64, 2816
    ws = [H.quantized(t, 40 + i, rows, cols) for i in range(4)]
    hs = [ctx.upload(w, t, rows, cols) for w in ws]
    xs = [Q.normal(60 + i, (cols,), 1.0) for i in range(3)]
    xd = [_dev(x) for x in xs]
    outs = torch.full((32, rows), float("nan"), device="cuda")
    ops = [dict(w=hs[i % 4], x=xd[i % 3], out=outs[i]) for i in range(32)]
    ctx.matvec_chain(ops)
    ctx.synchronize()
    got = outs.cpu().numpy()
    for i in range(32):
        ref = O.matvec_f64(t, ws[i % 4], rows, cols, xs[i % 3])
        assert O.max_rel_err(got[i], ref) < H.REPORT_TOL, i
    for h in hs:
        h.free()


def test_host_buffer_form_with_pinned_and_pageable_outputs(ctx):
    """LEV_FLAG_HOST_IO: inputs are copied in, one launch, outputs come back -- by the kernel's own stores when the
    output buffer is pinned host memory, by a copy otherwise.  Both give the bits of the device-pointer call, and
    the words after a pinned output stay untouched."""
    specs = [("q4_k", 96, 768), ("q6_k", 48, 3072), ("q4_0", 300, 2816)]
    hs, xs, refs = [], [], []
    for i, (name, rows, cols) in enumerate(specs):
        t = H.TYPES[name]
        w = H.quantized(t, 1200 + i, rows, cols)
        hs.append(ctx.upload(w, t, rows, cols))
        xs.append(Q.normal(1300 + i, (cols,), 1.0))
    dev_out = ctx.matvec_chain([dict(w=h, x=_dev(x), out=torch.empty(h.rows, device="cuda")) for h, x in zip(hs, xs)])
    ctx.synchronize()
    want = [o.cpu().numpy() for o in dev_out]
    pageable = [np.full(h.rows + 8, 7.0, np.float32) for h in hs]
    pinned = [torch.full((h.rows + 8,), 7.0).pin_memory() for h in hs]
    for outs in (pageable, [p.numpy() for p in pinned], [pageable[0], pinned[1].numpy(), pageable[2]]):
        for o in outs:
            o[:] = 7.0
        ctx.matvec_chain([dict(w=h, x=x, out=o[:h.rows]) for h, x, o in zip(hs, xs, outs)])
        for h, o, ref in zip(hs, outs, want):
            assert np.array_equal(o[:h.rows].view(np.uint32), ref.view(np.uint32))
            assert (o[h.rows:] == 7.0).all()
    # inputs: pinned ones are fetched by one small kernel, pageable ones by a queued copy each; a pinned input
    # rewritten by the host between two calls is read afresh (nothing is served from a cache)
    pin_x = [torch.from_numpy(x.copy()).pin_memory() for x in xs]
    outs = [p.numpy() for p in pinned]
    for ins in ([p.numpy() for p in pin_x], [pin_x[0].numpy(), xs[1], pin_x[2].numpy()]):
        for o in outs:
            o[:] = 7.0
        l0 = ctx.launch_count()
        ctx.matvec_chain([dict(w=h, x=x, out=o[:h.rows]) for h, x, o in zip(hs, ins, outs)])
        assert ctx.launch_count() - l0 == 2  # the fetch and the list
        for h, o, ref in zip(hs, outs, want):
            assert np.array_equal(o[:h.rows].view(np.uint32), ref.view(np.uint32))
    for rep in range(3):
        for p in pin_x:
            p.mul_(-0.5)
        ctx.matvec_chain([dict(w=h, x=p.numpy(), out=o[:h.rows]) for h, p, o in zip(hs, pin_x, outs)])
        again = ctx.matvec_chain([dict(w=h, x=p.cuda(), out=torch.empty(h.rows, device="cuda")) for h, p in zip(hs, pin_x)])
        ctx.synchronize()
        for h, o, ref in zip(hs, outs, again):
            assert np.array_equal(o[:h.rows].view(np.uint32), ref.cpu().numpy().view(np.uint32))
    for h in hs:
        h.free()


def test_chain_rejections(ctx):
    t = H.TYPES["q4_k"]
    w = H.quantized(t, 1, 32, 256)
    wh = ctx.upload(w, t, 32, 256)
    x = torch.zeros(256, device="cuda")
    y = torch.zeros(32, device="cuda")
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_chain([dict(w=wh, x=x, out=y, rows=64)])
    assert e.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_chain([dict(w=wh, x=x, out=x[:32])])
    assert e.value.name == "badArgument"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_chain([dict(w=wh, x=x, out=y)] * 33)
    assert e.value.name == "badArgument"
    wh.free()
