"""One rank of the multi-GPU parity check; launched by tests/test_gpu_dist.py
through torch.distributed.run (one process per GPU)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import leviathan_b200 as lev  # noqa: E402
from leviathan_b200 import dist as D  # noqa: E402
from leviathan_b200 import quant as Q  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = lev.Context(local)
    rank, world = D.init_from_torch(ctx)
    dev = f"cuda:{local}"

    # dense: rows split, y all-gathered
    for t, rows, cols, n_cols in ((Q.GGML_Q4_K, 64 * world, 1024, 1), (Q.GGML_Q4_0, 32 * world, 704, 3),
                                  (Q.GGML_Q6_K, 16 * world, 512, 2)):
        w = Q.quantized_normal(t, 11, rows, cols).numpy()
        x = Q.normal(12, (n_cols, cols), 1.0)
        r0, nr = D.row_shard(rows, rank, world)
        wh = ctx.upload(D.slice_blocks(w, t, rows, cols, r0, nr), t, nr, cols)
        y = ctx.matvec_rowsplit_allgather(wh, torch.from_numpy(x).to(dev), world).cpu().numpy()
        for c in range(n_cols):
            err = O.max_rel_err(y[c], O.matvec_f64(t, w, rows, cols, x[c]))
            assert err < 1e-4, ("rowsplit", t, c, err)
        wh.free()

    # a list of row-split products in one submission, twice (the heap halves alternate)
    specs = [(Q.GGML_Q4_K, 96 * world, 1024), (Q.GGML_Q4_K, 32 * world, 1024), (Q.GGML_Q6_K, 48 * world, 768)]
    ws, hs, xs = [], [], {}
    for j, (t, rows, cols) in enumerate(specs):
        w = Q.quantized_normal(t, 31 + j, rows, cols).numpy()
        r0, nr = D.row_shard(rows, rank, world)
        ws.append(w)
        hs.append(ctx.upload(D.slice_blocks(w, t, rows, cols, r0, nr), t, nr, cols))
        xs.setdefault(cols, Q.normal(40 + cols, (cols,), 1.0))
    xd = {c: torch.from_numpy(v).to(dev) for c, v in xs.items()}
    for rep in range(2):
        outs = [torch.full((rows,), float("nan"), device=dev) for _, rows, _ in specs]
        ctx.matvec_chain_rowsplit([dict(w=hs[j], x=xd[specs[j][2]], out=outs[j]) for j in range(len(specs))])
        for j, (t, rows, cols) in enumerate(specs):
            err = O.max_rel_err(outs[j].cpu().numpy(), O.matvec_f64(t, ws[j], rows, cols, xs[cols]))
            assert err < 1e-4, ("chain rowsplit", rep, j, err)
    for h in hs:
        h.free()

    peer = bool(ctx.lib.lev_dist_peer_memory(ctx.handle))
    if os.environ.get("LEV_EXPECT_PEER", "1") == "1":
        assert peer, "the ranks' heaps were not mapped into each other"

    # prefill GEMM: rows split, every rank ends with the whole Y (every 13th row against the rounded-operand oracle)
    t, rows, cols, tokens = Q.GGML_Q4_K, 192 * world, 1024, 96
    w = Q.quantized_normal(t, 21, rows, cols).numpy()
    xg = Q.normal(22, (tokens, cols), 1.0)
    r0, nr = D.row_shard(rows, rank, world)
    wh = ctx.upload(D.slice_blocks(w, t, rows, cols, r0, nr), t, nr, cols)
    xb = ctx.act_bf16(torch.from_numpy(xg).to(dev))
    for rep in range(3):  # consecutive calls alternate between the two halves of the heap
        yfull = ctx.gemm_prefill_rowsplit_allgather(wh, xb, world).cpu().numpy()
        ref = O.gemm_rounded_f64(t, w, rows, cols, xg, "bf16", 0, 13)
        err = O.max_rel_err(yfull[:, ::13], ref)
        assert err < 1e-3, ("rowsplit gemm", rep, err)
    wh.free()

    # MoE: experts sharded, tokens data-parallel
    e, h, i, k, t_local = 8 * world, 1056, 512, 5, 3
    g = torch.Generator().manual_seed(77)
    gu = Q.quantize_q4_0(torch.randn((e * 2 * i, h), generator=g) * 0.02).numpy()
    dn = Q.quantize_q4_0(torch.randn((e * h, i), generator=g) * 0.02).numpy()
    rw = (torch.randn((e, h), generator=g) * 0.02).numpy()
    x_all = Q.normal(78, (world * t_local, h), 1.0)
    first, count = D.expert_shard(e, rank, world)
    gs, ds = 2 * i * (h // 32) * 18, h * (i // 32) * 18
    mw = ctx.moe_upload(rw, gu[first * gs:(first + count) * gs], dn[first * ds:(first + count) * ds], e, h, i, first, count)
    x = torch.from_numpy(x_all[rank * t_local:(rank + 1) * t_local].copy()).to(dev)
    out, idx, wts = ctx.moe_layer(mw, x, k, want_routing=True, expert_parallel=True)
    out, idx, wts = out.cpu().numpy(), idx.cpu().numpy(), wts.cpu().numpy()
    for j in range(t_local):
        ri, rwt, _, ref64 = O.moe_token(h, i, e, k, rw, gu, dn, x_all[rank * t_local + j])
        assert np.array_equal(idx[j], ri), ("ep idx", j)
        assert np.max(np.abs(wts[j] - rwt)) <= 1e-6
        err = O.max_rel_err(out[j], ref64)
        assert err < 1e-4, ("ep out", j, err)
    # twice the same bits
    out2 = ctx.moe_layer(mw, x, k, expert_parallel=True).cpu().numpy()
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
    # and the bits of the single-GPU layer over the whole batch (every expert resident on this rank)
    if peer:
        mw_all = ctx.moe_upload(rw, gu, dn, e, h, i)
        one = ctx.moe_layer(mw_all, torch.from_numpy(x_all).to(dev), k).cpu().numpy()
        # decode-sized batches run on the streaming kernels, where a tile's K range is cut over the warps of a
        # block according to how many jobs the block has: no sum crosses a rank, but the f32 association inside
        # a row follows the (different) job lists, so the two agree to rounding, not to the bit
        mine = one[rank * t_local:(rank + 1) * t_local]
        assert O.max_rel_err(out, mine.astype(np.float64)) < 2e-6, "ep vs single GPU"
        mw_all.free()

    # the 128-expert top-8 layer of the benchmark at 256 tokens in all (2048 pairs: the tensor-core form)
    e2, h2, i2, k2 = 128, 2816, 704, 8
    t2 = 256 // world
    g2 = torch.Generator(device=dev).manual_seed(1234)
    gu2 = Q.quantize_q4_0(torch.randn((e2 * 2 * i2, h2), generator=g2, device=dev) * 0.02)
    dn2 = Q.quantize_q4_0(torch.randn((e2 * h2, i2), generator=g2, device=dev) * 0.02)
    rw2_d = torch.randn((e2, h2), generator=g2, device=dev) * 0.02
    rw2 = rw2_d.cpu().numpy()
    x2_all = Q.normal(79, (world * t2, h2), 1.0)
    f2, c2 = D.expert_shard(e2, rank, world)
    gs2, ds2 = 2 * i2 * (h2 // 32) * 18, h2 * (i2 // 32) * 18
    mw2 = ctx.moe_upload(rw2_d, gu2[f2 * gs2:(f2 + c2) * gs2], dn2[f2 * ds2:(f2 + c2) * ds2], e2, h2, i2, f2, c2)
    x2 = torch.from_numpy(x2_all[rank * t2:(rank + 1) * t2].copy()).to(dev)
    o2, idx2, _ = ctx.moe_layer(mw2, x2, k2, want_routing=True, expert_parallel=True)
    o2, idx2 = o2.cpu().numpy(), idx2.cpu().numpy()
    gu2h, dn2h = gu2.cpu().numpy(), dn2.cpu().numpy()
    for j in (0, t2 // 2, t2 - 1):
        ri, _, _, ref64 = O.moe_token(h2, i2, e2, k2, rw2, gu2h, dn2h, x2_all[rank * t2 + j])
        assert np.array_equal(idx2[j], ri), ("ep idx big", j)
        scale = max(1.0, float(np.max(np.abs(ref64))))
        assert float(np.max(np.abs(o2[j] - ref64))) / scale < 5e-3, ("ep out big", j)
    if peer:
        mw2_all = ctx.moe_upload(rw2_d, gu2, dn2, e2, h2, i2)
        one2 = ctx.moe_layer(mw2_all, torch.from_numpy(x2_all).to(dev), k2).cpu().numpy()
        assert np.array_equal(o2.view(np.uint32), one2[rank * t2:(rank + 1) * t2].view(np.uint32)), "ep != single GPU (tensor-core form)"
        mw2_all.free()
    mw2.free()
    torch.cuda.synchronize()
    dist.barrier()

    # the decode step on several GPUs: every rank decodes its own sequences, the experts are sharded; against the
    # same step with every expert resident, on the same caches and tokens, eager and as one CUDA graph
    from leviathan_b200.decoder import DecoderConfig, SyntheticDecoder

    cfg = DecoderConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=128, experts=8 * world, top_k=2, expert_inter=64,
                        vocab=512, positions=48, page=16)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        dec = SyntheticDecoder(ctx, cfg, batch=2, rank=rank, world=world)
        one = SyntheticDecoder(ctx, cfg, batch=2)
        for a, b in zip(one.layers, dec.layers):
            a.cache.k.copy_(b.cache.k)
            a.cache.v.copy_(b.cache.v)
        toks = torch.tensor([3 + 11 * rank, 40 + rank], dtype=torch.int32, device=dev)
        dec.tok.copy_(toks)
        one.tok.copy_(toks)
        one.step()
        dec.step()
        torch.cuda.synchronize()
        lo, le = one.logits.cpu().numpy(), dec.logits.cpu().numpy()
        assert float(np.max(np.abs(lo - le))) / max(1.0, float(np.max(np.abs(lo)))) < 1e-4, "decoder: expert-parallel step"
        assert np.array_equal(one.tok.cpu().numpy(), dec.tok.cpu().numpy()), "decoder: tokens"
        if peer:  # the peer-memory exchange keeps its epochs on the device, so the step replays as a graph
            dec.tok.copy_(toks)
            dec.capture()
            dist.barrier()
            dec.replay()
            torch.cuda.synchronize()
            assert np.array_equal(dec.logits.cpu().numpy().view(np.uint32), le.view(np.uint32)), "decoder: graph replay"
        dist.barrier()
        dec.free()
        one.free()
    mw.free()
    ctx.close()
    dist.destroy_process_group()
    print(f"rank {rank}/{world} OK", flush=True)


if __name__ == "__main__":
    main()
