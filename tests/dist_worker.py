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
    torch.cuda.synchronize()
    dist.barrier()
    mw.free()
    ctx.close()
    dist.destroy_process_group()
    print(f"rank {rank}/{world} OK", flush=True)


if __name__ == "__main__":
    main()
