"""Sharding rules of the multi-GPU paths (host-side logic, no device code).

Dense projections: output rows are split into equal contiguous slices, one
per rank, each a whole number of 16-row tiles; y is all-gathered.
MoE: experts are split into equal contiguous slices; tokens stay
data-parallel with the same count on every rank.
"""
from __future__ import annotations


def row_shard(rows: int, rank: int, world: int) -> tuple[int, int]:
    """(first_row, row_count) of `rank`; rows must split into equal 16-row-aligned slices."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if rows % world or (rows // world) % 16:
        raise ValueError(f"{rows} rows do not split into {world} slices of whole 16-row tiles")
    per = rows // world
    return rank * per, per


def expert_shard(experts: int, rank: int, world: int) -> tuple[int, int]:
    """(first_expert, expert_count) resident on `rank`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if experts % world:
        raise ValueError(f"{experts} experts do not split over {world} ranks")
    per = experts // world
    return rank * per, per


def expert_owner(expert: int, experts: int, world: int) -> int:
    return expert // (experts // world)


def slice_blocks(blocks, ggml_type: int, rows: int, cols: int, first: int, count: int):
    """Bytes of rows [first, first+count) of a row-major GGUF block tensor."""
    values, nbytes = {2: (32, 18), 12: (256, 144), 14: (256, 210)}[ggml_type]
    row_bytes = cols // values * nbytes
    return blocks[first * row_bytes:(first + count) * row_bytes]


def init_from_torch(ctx, group=None):
    """Create the context's NCCL communicator from a torch.distributed group:
    rank 0 makes the id, everyone receives it over the existing group."""
    import torch.distributed as dist

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [ctx.dist_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    ctx.dist_init(rank, world, box[0])
    return rank, world
