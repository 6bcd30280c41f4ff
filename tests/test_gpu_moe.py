"""Parity of the routed-MoE composite with the oracle, stage by stage and
end to end, through the C ABI."""
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


def make_moe(experts, hidden, inter, seed):
    """Seeded N(0, 0.02) experts (Q4_0) and router, generated and quantized on the GPU."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    gu = Q.quantize_q4_0(torch.randn((experts * 2 * inter, hidden), generator=g, device="cuda") * 0.02)
    dn = Q.quantize_q4_0(torch.randn((experts * hidden, inter), generator=g, device="cuda") * 0.02)
    rw = torch.randn((experts, hidden), generator=g, device="cuda") * 0.02
    return rw.cpu().numpy(), gu.cpu().numpy(), dn.cpu().numpy()


SHAPES = {
    # name: experts, hidden, inter, top_k
    "tail": (8, 96, 32, 3),          # tools/moe_lower/fixtures/tail-region.json
    "lanes": (16, 1056, 512, 5),     # Sources/leviathan-tests/main.swift:9031-9040 (33 blocks, slot tail)
    "gemma": (128, 2816, 704, 8),    # tools/moe_lower/fixtures/gemma4-26b-region.json
}


@pytest.fixture(scope="module")
def models(ctx):
    out = {}
    for name, (e, h, i, k) in SHAPES.items():
        rw, gu, dn = make_moe(e, h, i, 1000 + len(out))
        out[name] = dict(rw=rw, gu=gu, dn=dn, mw=ctx.moe_upload(rw, gu, dn, e, h, i), dims=(e, h, i, k))
    yield out
    for m in out.values():
        m["mw"].free()


@pytest.mark.parametrize("name,tokens", [("tail", 1), ("tail", 7), ("lanes", 5), ("gemma", 1), ("gemma", 32), ("gemma", 300), ("gemma", 130)])
def test_router_is_bit_exact(ctx, models, name, tokens):
    m = models[name]
    e, h, i, k = m["dims"]
    x = Q.normal(7 + tokens, (tokens, h), 1.0)
    idx, wts, scores = ctx.moe_route(m["mw"], torch.from_numpy(x).cuda(), k, want_scores=True, check_finite=True)
    idx, wts, scores = idx.cpu().numpy(), wts.cpu().numpy(), scores.cpu().numpy()
    min_gap = np.inf
    for t in range(tokens):
        ref_s = O.router_logits(m["rw"], x[t])
        assert np.array_equal(scores[t].view(np.uint32), ref_s.view(np.uint32)), (name, t)
        ref_i, ref_w = O.router_topk(ref_s, k)
        assert np.array_equal(idx[t], ref_i), (name, t)
        assert np.max(np.abs(wts[t] - ref_w)) <= 1e-6
        srt = np.sort(ref_s)[::-1]
        min_gap = min(min_gap, float(srt[k - 1] - srt[k]))
    print(f"router {name} T={tokens}: smallest rank-{k}/rank-{k + 1} logit gap {min_gap:.3e}")


def test_router_ties_go_to_the_lower_index(ctx, models):
    m = models["tail"]
    e, h, i, k = m["dims"]
    rw = np.zeros((e, h), np.float32)
    rw[2, 0] = rw[5, 0] = rw[1, 0] = 1.0   # three equal top scores
    rw[7, 1] = 0.5
    mw = ctx.moe_upload(rw, m["gu"], m["dn"], e, h, i)
    x = np.zeros((1, h), np.float32)
    x[0, 0], x[0, 1] = 2.0, 1.0
    idx, wts = ctx.moe_route(mw, x, 4)
    assert idx[0].tolist() == [1, 2, 5, 7]
    ref_i, ref_w = O.router_topk(O.router_logits(rw, x[0]), 4)
    assert np.array_equal(idx[0], ref_i) and np.max(np.abs(wts[0] - ref_w)) <= 1e-6
    mw.free()


@pytest.mark.parametrize("tokens,top_k,experts", [(1, 8, 128), (32, 8, 128), (512, 8, 128), (5, 3, 8), (9, 5, 16)])
def test_grouping_is_bit_exact(ctx, tokens, top_k, experts):
    rng = np.random.default_rng(tokens * 31 + top_k)
    idx = np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    counts, offsets, perm = ctx.moe_group(torch.from_numpy(idx).cuda(), experts)
    rc, ro, rp = O.group_tokens(idx, experts)
    assert np.array_equal(counts.cpu().numpy(), rc)
    assert np.array_equal(offsets.cpu().numpy(), ro)
    assert np.array_equal(perm.cpu().numpy(), rp)
    c2, o2, p2 = ctx.moe_group(idx, experts)  # host buffers
    assert np.array_equal(c2, rc) and np.array_equal(o2, ro) and np.array_equal(p2, rp)


def _region_ref(m, x_t, idx_t):
    e, h, i, k = m["dims"]
    gs, ds = 2 * i * (h // 32) * 18, h * (i // 32) * 18
    gu = np.concatenate([m["gu"][int(ex) * gs:(int(ex) + 1) * gs] for ex in idx_t])
    dn = np.concatenate([m["dn"][int(ex) * ds:(int(ex) + 1) * ds] for ex in idx_t])
    return O.moe_region_f64(h, i, len(idx_t), gu, dn, x_t)


@pytest.mark.parametrize("name,tokens", [("tail", 1), ("tail", 9), ("lanes", 6), ("gemma", 1), ("gemma", 32)])
def test_expert_ffn_matches_f64_region_oracle(ctx, models, name, tokens):
    m = models[name]
    e, h, i, k = m["dims"]
    x = Q.normal(90 + tokens, (tokens, h), 1.0)
    rng = np.random.default_rng(5 + tokens)
    idx = np.stack([rng.choice(e, k, replace=False) for _ in range(tokens)]).astype(np.int32)
    y, act = ctx.moe_experts(m["mw"], torch.from_numpy(x).cuda(), torch.from_numpy(idx).cuda(), want_act=True)
    y, act = y.cpu().numpy(), act.cpu().numpy()
    check = range(tokens) if tokens <= 9 else [0, tokens // 2, tokens - 1]
    for t in check:
        _, _, ract, rdn = _region_ref(m, x[t], idx[t])
        assert O.max_rel_err(act[t], ract) < H.REPORT_TOL, (name, t)
        assert O.max_rel_err(y[t], rdn) < H.REPORT_TOL, (name, t)
    # the same call again gives the same bits
    y2 = ctx.moe_experts(m["mw"], torch.from_numpy(x).cuda(), torch.from_numpy(idx).cuda()).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))


def test_hand_computed_region_on_the_gpu(ctx):
    """Sources/leviathan-tests/main.swift:8925-8946: gate 16, up 2, act 32, down 512."""
    blk = lambda lo, hi, q: [lo, hi] + [q] * 16
    gu, dn = [], []
    for _ in range(32):
        gu += blk(0x00, 0x3C, 0x98)
    for _ in range(32):
        gu += blk(0x00, 0x30, 0x98)
    for _ in range(32):
        dn += blk(0x00, 0x38, 0x99)
    rw = np.zeros((1, 32), np.float32)
    mw = ctx.moe_upload(rw, np.array(gu, np.uint8), np.array(dn, np.uint8), 1, 32, 32)
    x = np.ones((1, 32), np.float32)
    y, act = ctx.moe_experts(mw, x, np.zeros((1, 1), np.int32), want_act=True)
    assert np.all(act == 32.0) and np.all(y == 512.0)
    out, idx, wts = ctx.moe_layer(mw, x, 1, want_routing=True, check_finite=True)
    assert idx[0, 0] == 0 and wts[0, 0] == 1.0 and np.all(out == 512.0)
    mw.free()


def test_combine_is_rank_ordered(ctx):
    rng = np.random.default_rng(3)
    y = rng.standard_normal((6, 8, 96)).astype(np.float32) * 1e3
    w = rng.random((6, 8)).astype(np.float32)
    out = ctx.moe_combine(torch.from_numpy(y).cuda(), torch.from_numpy(w).cuda()).cpu().numpy()
    for t in range(6):
        assert np.array_equal(out[t].view(np.uint32), O.combine(y[t], w[t]).view(np.uint32))
    bad = w.copy()
    bad[0, 0] = np.nan
    with pytest.raises(lev.LevError) as e:
        ctx.moe_combine(y, bad)
    assert e.value.name == "nonFiniteInput"


@pytest.mark.parametrize("name,tokens", [("tail", 4), ("lanes", 3), ("gemma", 1), ("gemma", 32)])
def test_layer_matches_oracle(ctx, models, name, tokens):
    m = models[name]
    e, h, i, k = m["dims"]
    x = Q.normal(400 + tokens, (tokens, h), 1.0)
    buf, view = H.guarded(tokens * h)
    out, idx, wts = ctx.moe_layer(m["mw"], torch.from_numpy(x).cuda(), k, out=view.view(tokens, h), want_routing=True,
                                  check_finite=True)
    torch.cuda.synchronize()
    assert H.guards_intact(buf, tokens * h)
    out, idx, wts = out.cpu().numpy(), idx.cpu().numpy(), wts.cpu().numpy()
    check = range(tokens) if tokens <= 4 else [0, 13, tokens - 1]
    for t in check:
        ri, rw_, rout, rout64 = O.moe_token(h, i, e, k, m["rw"], m["gu"], m["dn"], x[t])
        assert np.array_equal(idx[t], ri)
        assert np.max(np.abs(wts[t] - rw_)) <= 1e-6
        assert O.max_rel_err(out[t], rout64) < H.REPORT_TOL, (name, t)
    # a token gives the same answer alone and inside a batch (to rounding: the column grouping differs)
    if tokens > 1:
        solo = ctx.moe_layer(m["mw"], torch.from_numpy(x[1:2]).cuda(), k).cpu().numpy()
        assert O.max_rel_err(solo[0], out[1].astype(np.float64)) < 1e-5
    # host-buffer entry
    hout = ctx.moe_layer(m["mw"], x, k)
    assert O.max_rel_err(hout[0], out[0].astype(np.float64)) < 1e-6


@pytest.mark.parametrize("tokens", [1, 3, 32])
def test_layer_with_folded_residual_gives_the_bits_of_layer_then_axpy(ctx, models, tokens):
    """lev_moe_layer_residual: out = residual + alpha * layer(x) from the combine launch, in place on the residual
    too; one launch fewer than the layer followed by lev_axpy, the same bits."""
    m = models["gemma"]
    e, h, i, k = m["dims"]
    x = torch.from_numpy(Q.normal(700 + tokens, (tokens, h), 1.0)).cuda()
    r = torch.from_numpy(Q.normal(710 + tokens, (tokens, h), 1.0)).cuda()
    for alpha in (1.0, -0.375):
        l0 = ctx.launch_count()
        want = ctx.axpy(alpha, ctx.moe_layer(m["mw"], x, k), r, out=torch.empty_like(r))
        separate = ctx.launch_count() - l0
        l0 = ctx.launch_count()
        got = ctx.moe_layer_residual(m["mw"], x, k, r, alpha, out=torch.empty_like(r))
        assert ctx.launch_count() - l0 == separate - 1
        ctx.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        inplace = r.clone()
        ctx.moe_layer_residual(m["mw"], x, k, inplace, alpha)
        ctx.synchronize()
        assert torch.equal(inplace.view(torch.int32), want.view(torch.int32))
    with pytest.raises(lev.LevError):
        ctx.moe_layer_residual(m["mw"], x, k, r, 1.0, out=x)
    with pytest.raises(lev.LevError):
        ctx.moe_layer_residual(m["mw"], x, k, r, float("nan"))


@pytest.mark.parametrize("tokens", [96, 512])
def test_prefill_sized_layer_runs_on_the_tensor_cores(ctx, models, tokens):
    """96 tokens x top-8 = 768 pairs and the 512-token batch (4096 pairs): the expert FFN runs as a
    grouped bf16 dequant-GEMM (tcgen05); routing stays bit-exact, outputs are held to the 2e-2 bar of
    tensor-core prefill and reported against 5e-3."""
    m = models["gemma"]
    e, h, i, k = m["dims"]
    x = Q.normal(777, (tokens, h), 1.0)
    buf, view = H.guarded(tokens * h)
    out, idx, wts = ctx.moe_layer(m["mw"], torch.from_numpy(x).cuda(), k, out=view.view(tokens, h), want_routing=True,
                                  check_finite=True)
    torch.cuda.synchronize()
    assert H.guards_intact(buf, tokens * h)
    out, idx = out.cpu().numpy(), idx.cpu().numpy()
    worst = 0.0
    sample = (0, 41, tokens - 1) if tokens < 512 else (0, 41, 95, 127, 255, 300, 400, 511)
    for t in sample:
        ri, _, _, rout64 = O.moe_token(h, i, e, k, m["rw"], m["gu"], m["dn"], x[t])
        assert np.array_equal(idx[t], ri)
        scale = max(1.0, float(np.max(np.abs(rout64))))
        worst = max(worst, float(np.max(np.abs(out[t] - rout64))) / scale, O.max_rel_err(out[t], rout64))
    print(f"moe layer T={tokens} on the tensor cores: worst error vs f64 oracle {worst:.3e}")
    assert worst < 2e-2, worst
    assert worst < 5e-3, worst
    out2 = ctx.moe_layer(m["mw"], torch.from_numpy(x).cuda(), k).cpu().numpy()
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))


def test_layer_after_release_of_the_gguf_copies(ctx, models):
    """A decode-only host drops the GGUF-order copies of the experts: decode-sized calls give the same bits as
    before, and a batch of 768 pairs, which would have gone to the tensor cores, runs on the f32-activation
    stream kernels instead (1e-4 of the f64 oracle instead of 5e-3)."""
    m = models["gemma"]
    e, h, i, k = m["dims"]
    mw = ctx.moe_upload(m["rw"], m["gu"], m["dn"], e, h, i)
    x1 = torch.from_numpy(Q.normal(801, (3, h), 1.0)).cuda()
    before = ctx.moe_layer(mw, x1, k).cpu().numpy()
    mw.release_gguf()
    after = ctx.moe_layer(mw, x1, k).cpu().numpy()
    assert np.array_equal(before.view(np.uint32), after.view(np.uint32))
    x = Q.normal(802, (96, h), 1.0)
    out = ctx.moe_layer(mw, torch.from_numpy(x).cuda(), k).cpu().numpy()
    for t in (0, 50, 95):
        _, _, _, rout64 = O.moe_token(h, i, e, k, m["rw"], m["gu"], m["dn"], x[t])
        assert float(np.max(np.abs(out[t] - rout64))) / max(1.0, float(np.max(np.abs(rout64)))) < 1e-4, t
    mw.free()


def test_moe_rejections(ctx, models):
    m = models["tail"]
    e, h, i, k = m["dims"]
    with pytest.raises(lev.LevError) as err:
        ctx.moe_upload(m["rw"], m["gu"][:-18], m["dn"], e, h, i)
    assert err.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as err:
        ctx.moe_upload(m["rw"], m["gu"], m["dn"], e, h + 1, i)
    assert err.value.name == "badDimensions"
    x = np.zeros((2, h), np.float32)
    with pytest.raises(lev.LevError) as err:
        ctx.moe_layer(m["mw"], x, e + 1)
    assert err.value.name == "badDimensions"
    x[1, 3] = np.inf
    with pytest.raises(lev.LevError) as err:
        ctx.moe_layer(m["mw"], x, k, check_finite=True)
    assert err.value.name == "nonFiniteInput"
    with pytest.raises(lev.LevError) as err:
        ctx.moe_experts(m["mw"], np.zeros((1, h), np.float32), np.array([[0, 1, e]], np.int32))
    assert err.value.name == "badArgument"
    bad = m["gu"].copy()
    bad[1] = 0x7C
    with pytest.raises(lev.LevError) as err:
        ctx.moe_upload(m["rw"], bad, m["dn"], e, h, i)
    assert err.value.name == "nonFiniteScale"
