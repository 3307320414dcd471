"""How the paths are split over the GPUs of one node.

Every path shards without an exchange step (no collective in the timed region):
GEMM by rows of A / C / D with B replicated, DLRM by batch, GEMV by rows.  A shard is
a contiguous range; ranges are aligned so that seeded inputs regenerate per shard
(rocwmma_b200.synth.CHUNK_ROWS) and so that packed DLRM rows stay 16-byte aligned.
"""
from __future__ import annotations

from .synth import CHUNK_ROWS


def row_range(total: int, world: int, rank: int, align: int = CHUNK_ROWS):
    """(first, count) of rank's contiguous share of `total` rows: equal shares rounded up to
    `align`, the last ranks may get fewer (or none)."""
    assert 0 <= rank < world
    per = -(-total // world)
    per = -(-per // align) * align
    first = min(total, rank * per)
    return first, max(0, min(per, total - first))


def gemm_shard(m: int, world: int, rank: int):
    """Rows of A, C and D owned by `rank` (B is replicated)."""
    return row_range(m, world, rank, CHUNK_ROWS)


def dlrm_shard(batch: int, world: int, rank: int):
    """Samples owned by `rank`; multiples of 8 keep the packed rows 16-byte aligned."""
    return row_range(batch, world, rank, 8)


def gemv_shard(m: int, world: int, rank: int):
    """Rows of A and y owned by `rank`; each rank holds its own column-major block with
    lda = its row count, x is replicated.  Multiples of 64 rows (one thread block's share)."""
    return row_range(m, world, rank, 64)


def max_over_ranks(value: float, device=None) -> float:
    """Slowest rank's time (torch.distributed must be initialised when world > 1)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
