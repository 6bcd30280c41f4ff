"""World-size-2 gloo ranks on CPU: the sharding rules and the expert-parallel
decomposition (all-gather tokens, replicated routing, local experts, summed
partials) reproduce the single-process oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from leviathan_b200 import dist as D
from leviathan_b200 import quant as Q

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rules():
    assert D.row_shard(12288, 3, 8) == (4608, 1536)
    assert D.expert_shard(128, 7, 8) == (112, 16)
    assert D.expert_owner(33, 128, 8) == 2
    with pytest.raises(ValueError):
        D.row_shard(4096 + 16, 0, 8)
    with pytest.raises(ValueError):
        D.row_shard(48, 0, 2)  # 24 rows per rank is not a whole number of 16-row tiles
    with pytest.raises(ValueError):
        D.expert_shard(10, 0, 4)
    blocks = np.arange(4 * 2 * 18, dtype=np.uint8)
    assert D.slice_blocks(blocks, 2, 4, 64, 1, 2).tolist() == list(range(36, 108))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    e, h, i, k, t_local = 8, 96, 32, 3, 2
    g = torch.Generator().manual_seed(5)
    gu = Q.quantize_q4_0(torch.randn((e * 2 * i, h), generator=g) * 0.02).numpy()
    dn = Q.quantize_q4_0(torch.randn((e * h, i), generator=g) * 0.02).numpy()
    rw = (torch.randn((e, h), generator=g) * 0.02).numpy()
    x_all = Q.normal(9, (world * t_local, h), 1.0)
    x = torch.from_numpy(x_all[rank * t_local:(rank + 1) * t_local].copy())
    # dispatch: all-gather of the token rows
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    gathered = torch.cat(parts).numpy()
    assert np.array_equal(gathered, x_all)
    first, count = D.expert_shard(e, rank, world)
    gs, ds = 2 * i * (h // 32) * 18, h * (i // 32) * 18
    partial = np.zeros((world * t_local, h), np.float32)
    for t in range(world * t_local):
        idx, wts = O.router_topk(O.router_logits(rw, gathered[t]), k)
        ys = np.zeros((k, h), np.float32)
        for r, ex in enumerate(idx):
            if first <= ex < first + count:
                assert D.expert_owner(int(ex), e, world) == rank
                _, _, _, d = O.moe_region_f64(h, i, 1, gu[ex * gs:(ex + 1) * gs], dn[ex * ds:(ex + 1) * ds], gathered[t])
                ys[r] = d[0].astype(np.float32)
        partial[t] = O.combine(ys, wts)
    # combine: sum of the ranks' partials, each rank keeps its own tokens
    total = torch.from_numpy(partial)
    dist.all_reduce(total)
    mine = total[rank * t_local:(rank + 1) * t_local].numpy()
    for j in range(t_local):
        _, _, ref, ref64 = O.moe_token(h, i, e, k, rw, gu, dn, x_all[rank * t_local + j])
        assert O.max_rel_err(mine[j], ref64) < 1e-5
    # dense: row split + all-gather
    rows, cols = 64, 256
    w = Q.quantized_normal(Q.GGML_Q4_K, 3, rows, cols).numpy()
    xv = Q.normal(4, (cols,), 1.0)
    r0, nr = D.row_shard(rows, rank, world)
    yl = torch.from_numpy(O.q4_k_matvec_f32(D.slice_blocks(w, Q.GGML_Q4_K, rows, cols, r0, nr), nr, cols, xv))
    ys = [torch.empty_like(yl) for _ in range(world)]
    dist.all_gather(ys, yl)
    assert np.array_equal(torch.cat(ys).numpy(), O.q4_k_matvec_f32(w, rows, cols, xv))
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")


def test_expert_parallel_and_row_split_decomposition_world2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
