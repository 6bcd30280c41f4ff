"""Decode attention over a paged KV cache (lev_attn_decode, lev_kv_append) against the f64 oracle.
The cache is filled through lev_kv_append with blocks handed out in a shuffled order, so block-table
indirection, fp16 storage and the append kernel are all on the tested path."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4  # max |got - ref| / max(1, |ref|), the f32-path report bar


@pytest.fixture(scope="module")
def ctx():
    c = lev.Context(0)
    yield c
    c.close()


def fill(ctx, cache, slot, tokens, kv_heads, hd, seed, chunk=64):
    """Appends `tokens` positions of seeded K, V to sequence `slot`; returns them as stored (after the
    cache's rounding), [tokens][kv_heads][hd] f32."""
    k = Q.normal(seed, (tokens, kv_heads, hd), 1.0).astype(np.float32) * np.float32(0.25)
    v = Q.normal(seed + 1, (tokens, kv_heads, hd), 1.0).astype(np.float32)
    for p in range(tokens):
        cache.ensure(slot, p)
    for t0 in range(0, tokens, chunk):
        n = min(chunk, tokens - t0)
        sl = torch.full((n,), slot, dtype=torch.int32, device="cuda")
        ps = torch.arange(t0, t0 + n, dtype=torch.int32, device="cuda")
        ctx.kv_append(cache, sl, ps, torch.from_numpy(k[t0:t0 + n]).cuda(), torch.from_numpy(v[t0:t0 + n]).cuda())
    if cache.k.dtype == torch.float16:
        k, v = k.astype(np.float16).astype(np.float32), v.astype(np.float16).astype(np.float32)
    return k, v


def shuffled(cache, seed):
    rng = np.random.default_rng(seed)
    rng.shuffle(cache.free)
    return cache


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("q_heads,kv_heads,hd", [(16, 8, 256), (4, 4, 128), (8, 2, 128), (8, 8, 256)])
def test_matches_the_f64_oracle(ctx, dtype, q_heads, kv_heads, hd):
    tokens, page = 1100, 16
    cache = shuffled(lev.PagedKV(128, page, kv_heads, hd, slots=3, max_blocks=80, dtype=dtype), 5)
    k, v = fill(ctx, cache, 1, tokens, kv_heads, hd, 40 + hd)
    # the stored cache reads back as appended
    flat = cache.ensure(1, 777)
    got_row = cache.k.reshape(-1, kv_heads, hd)[flat].float().cpu().numpy()
    assert np.array_equal(got_row, k[777])
    q = Q.normal(7, (1, q_heads, hd), 1.0).astype(np.float32)
    slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    for qpos in (0, 1, 15, 16, 17, 63, 500, tokens - 1):
        for window, scale in ((0, 1.0), (0, hd ** -0.5), (256, 1.0), (1, 1.0)):
            pos = torch.tensor([qpos], dtype=torch.int32, device="cuda")
            got = ctx.attn_decode(cache, slot, pos, torch.from_numpy(q).cuda(), window, scale).cpu().numpy()[0]
            ref = O.attention_f64(q[0], k[:qpos + 1], v[:qpos + 1], window, scale)
            assert O.max_rel_err(got.reshape(-1), ref.reshape(-1)) < TOL, (dtype, q_heads, kv_heads, hd, qpos, window, scale)
    ctx.synchronize()


def test_columns_of_different_sequences_and_repeat_runs(ctx):
    q_heads, kv_heads, hd = 16, 8, 256
    cache = shuffled(lev.PagedKV(160, 16, kv_heads, hd, slots=4, max_blocks=64, dtype="f16"), 9)
    lens = {0: 1000, 2: 37, 3: 513}
    kv = {s: fill(ctx, cache, s, n, kv_heads, hd, 100 + s) for s, n in lens.items()}
    cols = [(0, 999), (2, 36), (3, 512), (0, 400), (3, 0)]
    q = Q.normal(8, (len(cols), q_heads, hd), 1.0).astype(np.float32)
    slot = torch.tensor([c[0] for c in cols], dtype=torch.int32, device="cuda")
    pos = torch.tensor([c[1] for c in cols], dtype=torch.int32, device="cuda")
    qd = torch.from_numpy(q).cuda()
    got = ctx.attn_decode(cache, slot, pos, qd, 0, 1.0).cpu().numpy()
    for c, (s, p) in enumerate(cols):
        ref = O.attention_f64(q[c], kv[s][0][:p + 1], kv[s][1][:p + 1], 0, 1.0)
        assert O.max_rel_err(got[c].reshape(-1), ref.reshape(-1)) < TOL, (c, s, p)
    again = ctx.attn_decode(cache, slot, pos, qd, 0, 1.0).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))  # fixed merge order: same bits
    # one column alone gives the bits it gave inside the batch
    alone = ctx.attn_decode(cache, slot[1:2], pos[1:2], qd[1:2].contiguous(), 0, 1.0).cpu().numpy()
    assert O.max_rel_err(alone[0].reshape(-1), got[1].astype(np.float64).reshape(-1)) < 1e-6
    # lev_attn_decode_ld: the same queries as the leading part of the rows of a fused [q | k | v] matrix
    fused = torch.full((len(cols), (q_heads + 2 * kv_heads) * hd), float("nan"), device="cuda")
    fused[:, :q_heads * hd] = qd.view(len(cols), -1)
    strided = ctx.attn_decode_fused_rows(cache, slot, pos, fused, q_heads, 0, 1.0).cpu().numpy()
    assert np.array_equal(strided.view(np.uint32), got.view(np.uint32))
    with pytest.raises(lev.LevError):
        ctx.attn_decode_fused_rows(cache, slot, pos, fused[:, :q_heads * hd - 2].contiguous(), q_heads, 0, 1.0)


def test_closed_forms_on_the_gpu(ctx):
    q_heads, kv_heads, hd = 4, 2, 128
    cache = lev.PagedKV(8, 16, kv_heads, hd, slots=1, max_blocks=4, dtype="f32")
    T = 40
    for p in range(T):
        cache.ensure(0, p)
    k = torch.ones((T, kv_heads, hd), device="cuda")
    v = torch.randn((T, kv_heads, hd), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    sl = torch.zeros(T, dtype=torch.int32, device="cuda")
    ps = torch.arange(T, dtype=torch.int32, device="cuda")
    ctx.kv_append(cache, sl, ps, k, v)
    q = torch.randn((1, q_heads, hd), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    out = ctx.attn_decode(cache, sl[:1], ps[-1:], q, 0, 1.0).cpu().numpy()[0]
    mean = v.double().mean(dim=0).cpu().numpy()
    for h in range(q_heads):  # equal keys: the mean of V of KV head h // 2
        assert O.max_rel_err(out[h], mean[h // 2]) < 1e-6
    one = ctx.attn_decode(cache, sl[:1], ps[:1], q, 0, 1.0).cpu().numpy()[0]
    assert np.array_equal(one[3], v[0, 1].cpu().numpy())  # a single position: its V row exactly


def test_indices_outside_the_layout_are_not_followed(ctx):
    q_heads, kv_heads, hd = 4, 4, 128
    cache = lev.PagedKV(8, 16, kv_heads, hd, slots=2, max_blocks=4, dtype="f16")
    fill(ctx, cache, 0, 20, kv_heads, hd, 3)
    q = torch.ones((2, q_heads, hd), device="cuda")
    good = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
    for slot, pos in (([0, 7], [5, 5]), ([0, 0], [5, 64]), ([0, -1], [5, 5]), ([0, 0], [5, -3])):
        out = ctx.attn_decode(cache, torch.tensor(slot, dtype=torch.int32, device="cuda"),
                              torch.tensor(pos, dtype=torch.int32, device="cuda"), q, 0, 1.0).cpu().numpy()
        assert np.all(np.isfinite(out[0])) and np.all(np.isnan(out[1]))
        with pytest.raises(lev.LevError) as e:
            ctx.synchronize()
        assert e.value.name == "badDimensions"
    # a block-table entry beyond the pool
    cache.table[0, 0] = 99
    out = ctx.attn_decode(cache, good, torch.tensor([5, 5], dtype=torch.int32, device="cuda"), q, 0, 1.0)
    with pytest.raises(lev.LevError):
        ctx.synchronize()
    ctx.synchronize()  # the record is cleared by the read
    # host-side rejections
    pos = torch.tensor([5, 5], dtype=torch.int32, device="cuda")
    with pytest.raises(lev.LevError) as e:
        ctx.attn_decode(cache, good, pos, torch.ones((2, 6, hd), device="cuda"), 0, 1.0)  # 6 heads over 4 KV heads
    assert e.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as e:
        ctx.attn_decode(cache, good, pos, q, -1, 1.0)
    assert e.value.name == "badArgument"
    bad = lev.PagedKV(8, 16, 4, 64, slots=1, max_blocks=4)
    with pytest.raises(lev.LevError) as e:
        ctx.attn_decode(bad, good[:1], pos[:1], torch.ones((1, 4, 64), device="cuda"), 0, 1.0)
    assert e.value.name == "unsupported"


def test_full_size_context(ctx):
    """The measured configuration: 16 query heads, 8 KV heads, head dimension 256, 4096 cached positions,
    fp16 pages of 16 handed out in a shuffled order; full attention and the model's 1024 window."""
    q_heads, kv_heads, hd, tokens = 16, 8, 256, 4096
    cache = shuffled(lev.PagedKV(tokens // 16 + 1, 16, kv_heads, hd, slots=1, max_blocks=tokens // 16, dtype="f16"), 11)
    k, v = fill(ctx, cache, 0, tokens, kv_heads, hd, 77, chunk=512)
    q = Q.normal(78, (1, q_heads, hd), 1.0).astype(np.float32)
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([tokens - 1], dtype=torch.int32, device="cuda")
    for window in (0, 1024):
        got = ctx.attn_decode(cache, slot, pos, torch.from_numpy(q).cuda(), window, 1.0).cpu().numpy()[0]
        ref = O.attention_f64(q[0], k, v, window, 1.0)
        assert np.all(np.isfinite(got))
        assert O.max_rel_err(got.reshape(-1), ref.reshape(-1)) < TOL, window
    # linearity in V: doubling every cached V row doubles the output exactly (powers of two are exact in fp16)
    base = ctx.attn_decode(cache, slot, pos, torch.from_numpy(q).cuda(), 0, 1.0).cpu().numpy()
    cache.v.mul_(2.0)
    twice = ctx.attn_decode(cache, slot, pos, torch.from_numpy(q).cuda(), 0, 1.0).cpu().numpy()
    assert np.array_equal(twice, 2.0 * base)
    ctx.synchronize()


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_many_columns_take_one_range_each(ctx, dtype):
    """Enough (column, KV head) pairs to fill the GPU: every pair is one range and writes its output
    itself (no partials, no merge launch)."""
    q_heads, kv_heads, hd, tokens, cols = 16, 8, 256, 300, 40
    cache = shuffled(lev.PagedKV(32, 16, kv_heads, hd, slots=2, max_blocks=24, dtype=dtype), 13)
    k, v = fill(ctx, cache, 1, tokens, kv_heads, hd, 90)
    q = Q.normal(91, (cols, q_heads, hd), 1.0).astype(np.float32)
    positions = [(7 * c + 3) % tokens for c in range(cols)]
    slot = torch.ones(cols, dtype=torch.int32, device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    l0 = ctx.launch_count()
    got = ctx.attn_decode(cache, slot, pos, torch.from_numpy(q).cuda(), 0, 1.0).cpu().numpy()
    assert ctx.launch_count() - l0 == 1
    for c in (0, 1, 17, cols - 1):
        ref = O.attention_f64(q[c], k[:positions[c] + 1], v[:positions[c] + 1], 0, 1.0)
        assert O.max_rel_err(got[c].reshape(-1), ref.reshape(-1)) < TOL, c
    ctx.synchronize()


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_norm_rope_append_in_one_launch_equals_the_two_calls(ctx, dtype):
    q_heads, kv_heads, hd, cols = 16, 8, 256, 3
    a = lev.PagedKV(16, 16, kv_heads, hd, slots=2, max_blocks=8, dtype=dtype)
    b = lev.PagedKV(16, 16, kv_heads, hd, slots=2, max_blocks=8, dtype=dtype)
    positions = [37, 5, 100]
    for cache in (a, b):
        for p in positions:
            cache.ensure(1, p)
    x = Q.normal(55, (cols, (q_heads + 2 * kv_heads) * hd), 1.0).astype(np.float32)
    qw = torch.from_numpy((1.0 + Q.normal(56, (hd,), 0.1)).astype(np.float32)).cuda()
    inv = torch.from_numpy((10000.0 ** (-np.arange(hd // 2, dtype=np.float64) / (hd // 2))).astype(np.float32)).cuda()
    slot = torch.ones(cols, dtype=torch.int32, device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    xa, xb = torch.from_numpy(x).cuda(), torch.from_numpy(x).cuda()
    ctx.qkv_norm_rope(xa, q_heads, kv_heads, hd, qw, qw, 1e-6, inv, pos)
    kv = xa.view(cols, q_heads + 2 * kv_heads, hd)
    ctx.kv_append(a, slot, pos, kv[:, q_heads:q_heads + kv_heads], kv[:, q_heads + kv_heads:])
    l0 = ctx.launch_count()
    ctx.qkv_norm_rope_append(xb, q_heads, b, slot, pos, qw, qw, 1e-6, inv)
    assert ctx.launch_count() - l0 == 1
    assert torch.equal(xa, xb) and torch.equal(a.k, b.k) and torch.equal(a.v, b.v)
    assert float(b.k.float().abs().sum()) > 0
    ctx.synchronize()
    # a position outside the table is recorded, not followed
    bad = torch.tensor([37, 5, 4096], dtype=torch.int32, device="cuda")
    ctx.qkv_norm_rope_append(torch.from_numpy(x).cuda(), q_heads, b, slot, bad, qw, qw, 1e-6, inv)
    with pytest.raises(lev.LevError):
        ctx.synchronize()
