"""One process per GPU: how the path is divided between ranks.

Hyrax rows (and whole layers) are independent, so ranks need no data-path collective: every rank
commits a contiguous block of rows with the generator table replicated in its own HBM, and only the
96-byte row commitments are gathered (``torch.distributed`` all-gather; NCCL on GPUs, gloo in the
CPU tests).  Timing across ranks is the maximum of the per-rank device times.
"""
from __future__ import annotations

import numpy as np


def row_block(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [start, end) of `rows` rows owned by `rank`; the first `rows % world` ranks
    hold one row more."""
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_rows(local: np.ndarray, rows: int, dist=None, device: str = "cpu") -> np.ndarray:
    """All-gather of per-rank row records (uint32[block_rows, k]) into uint32[rows, k], in row order.
    `dist` is the initialised ``torch.distributed`` module (None = single process)."""
    local = np.ascontiguousarray(local, dtype=np.uint32)
    if dist is None or dist.get_world_size() == 1:
        assert local.shape[0] == rows
        return local
    import torch
    world, rank = dist.get_world_size(), dist.get_rank()
    k = local.shape[1]
    longest = row_block(rows, 0, world)[1]
    padded = np.zeros((longest, k), dtype=np.int64)      # int64 payload: every backend supports it
    padded[: local.shape[0]] = local
    mine = torch.from_numpy(padded).to(device)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    out = np.empty((rows, k), dtype=np.uint32)
    for r, p in enumerate(parts):
        s, e = row_block(rows, r, world)
        out[s:e] = p.cpu().numpy()[: e - s].astype(np.uint32)
    assert row_block(rows, rank, world)[1] - row_block(rows, rank, world)[0] == local.shape[0]
    return out


def commit_rows_sharded(scalars: np.ndarray, wd: int, commit_fn, dist=None, device: str = "cpu") -> np.ndarray:
    """Row commitments of a host int32 tensor with the rows dealt to the ranks in contiguous blocks.
    `commit_fn(block_scalars) -> uint32[block_rows, 24]` commits one block on this rank's GPU
    (e.g. ``lambda s: commit_i32_host(ctx, table, s, wd)``)."""
    scalars = np.ascontiguousarray(scalars, dtype=np.int32).reshape(-1)
    rows = scalars.size // wd
    world = 1 if dist is None else dist.get_world_size()
    rank = 0 if dist is None else dist.get_rank()
    s, e = row_block(rows, rank, world)
    local = commit_fn(scalars[s * wd:e * wd]) if e > s else np.zeros((0, 24), dtype=np.uint32)
    return gather_rows(local, rows, dist, device)


def max_over_ranks(value: float, dist=None, device: str = "cpu") -> float:
    """Maximum of a per-rank timing (the number multi-GPU throughput is computed from)."""
    if dist is None or dist.get_world_size() == 1:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
