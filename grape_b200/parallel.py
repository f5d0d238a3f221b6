"""One process per GPU: how the path is divided between ranks.

Hyrax rows (and whole layers) are independent, so ranks need no data-path collective: every rank
commits a contiguous block of rows with the generator table replicated in its own HBM, and only the
96-byte row commitments are gathered (``torch.distributed`` all-gather; NCCL on GPUs, gloo in the
CPU tests).  Timing across ranks is the maximum of the per-rank device times.

The matrix-product sumcheck can also be split: the inner dimension is dealt to the ranks by residue
class, every rank runs the rounds that stay inside its shard, and a single small all-gather carries
the per-round partial sums (``prove_matmul_sharded``).
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


class _DeviceBytes:
    """A device region as a CUDA-array-interface object (bytes), so that torch can wrap it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False),
                                         "version": 2, "strides": None}


def torch_view(ptr: int, nbytes: int):
    """torch uint8 tensor over `nbytes` of device memory at `ptr` (no copy; the caller keeps it alive)."""
    import torch
    return torch.as_tensor(_DeviceBytes(ptr, nbytes), device="cuda")


def library_stream(ctx):
    """The context's CUDA stream as a torch stream: collectives issued under ``torch.cuda.stream(...)``
    of it are ordered after the library's kernels and before its next ones on the device, with no
    host synchronisation in between."""
    import torch
    return torch.cuda.ExternalStream(ctx.stream)


def gather_rows_device(ctx, d_local, block_rows: int, d_all, dist, record_bytes: int = 96):
    """NCCL all-gather of this rank's `block_rows` row commitments (device buffer `d_local`) into the
    device buffer `d_all` ([world][block_rows] records, rank order), issued on the library's stream.
    Every rank passes the same `block_rows` (``row_block(rows, 0, world)`` length; ranks with one row
    fewer pad their last record).  Nothing passes through the host."""
    import torch
    from .host import _p
    world = dist.get_world_size()
    n = block_rows * record_bytes
    src = torch_view(_p(d_local), n)
    dst = torch_view(_p(d_all), n * world)
    with torch.cuda.stream(library_stream(ctx)):
        dist.all_gather_into_tensor(dst, src)


def commit_rows_sharded_device(ctx, table, d_scalars_block, block_rows: int, wd: int, d_local, d_all, dist,
                               max_bits: int = 32):
    """One rank's share of a row commitment dealt to the GPUs (Hyrax::commit over a row block,
    src/Hyrax.cu:312-333, rows are independent): commit `block_rows` rows of `wd` int32 scalars resident
    at `d_scalars_block` into `d_local`, then all-gather every rank's records into `d_all` over NCCL.
    All work is queued on the library's stream; the caller synchronises when it needs the result."""
    from .host import commit_i32
    commit_i32(ctx, table, d_scalars_block, block_rows * wd, wd, d_local, max_bits=max_bits)
    if dist is not None and dist.get_world_size() > 1:
        gather_rows_device(ctx, d_local, block_rows, d_all, dist, table.jacobian_bytes)


def hyrax_open_sharded(ctx, table, d_block, block_rows: int, rows: int, N: int, eval_point, c: int, G_jacobian, dist=None,
                       z_out=None):
    """``Hyrax::open`` (src/Hyrax.cu:237-305) of ONE layer's tensor whose `rows` commitment rows (of
    wd = N * 16 field elements) are dealt to the ranks in contiguous blocks of `block_rows`; `d_block` is
    this rank's block on its GPU.  The reference folds the row variables of the whole tensor on one GPU
    (src/Hyrax.cu:263-279); here every rank folds its own rows over the low row variables, ONE all-gather
    carries the wd-element partial vectors (NCCL, on the library's stream), every rank folds the gathered
    [ranks][wd] tensor over the remaining (high) row variables, and the opening proper (blinding vector,
    z, com_d, com_ad) runs on that single row.  Same proof as the unsharded call with the same random
    stream.  `rows`, `block_rows` and the number of ranks must be powers of two."""
    import torch
    from . import host
    from .host import COM_SCALE, _p
    world = 1 if dist is None else dist.get_world_size()
    wd = N * COM_SCALE
    if block_rows * world != rows or rows & (rows - 1) or world & (world - 1):
        raise ValueError("rows = ranks * block_rows, all powers of two")
    lw = max(wd - 1, 0).bit_length()
    l_local = max(block_rows - 1, 0).bit_length()
    e = list(eval_point)
    if len(e) != lw + max(rows - 1, 0).bit_length():
        raise ValueError("the evaluation point must have log2(rows * wd) coordinates")
    d_e = ctx.fr_upload(e)
    d_part = ctx.alloc(wd * 32)
    if block_rows > 1:
        ctx.fr_fold(d_block, block_rows * wd, d_e.at(lw * 32), block_rows, wd, d_part)
    else:
        ctx._check(ctx.lib.grape_d2d(ctx.handle, d_part.ptr, _p(d_block), wd * 32))
    if world > 1:
        d_all = ctx.alloc(world * wd * 32)
        with torch.cuda.stream(library_stream(ctx)):
            dist.all_gather_into_tensor(torch_view(d_all.ptr, world * wd * 32), torch_view(d_part.ptr, wd * 32))
        d_x = ctx.alloc(wd * 32)
        ctx.fr_fold(d_all, world * wd, d_e.at((lw + l_local) * 32), world, wd, d_x)
    else:
        d_x = d_part
    return host.hyrax_open(ctx, table, d_x, wd, N, 1, e[:lw], c, G_jacobian, z_out=z_out)


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


def shard_columns(t: np.ndarray, K: int, rank: int, world: int) -> np.ndarray:
    """Residue-class shard of the last axis: ``t`` viewed as [..., K] -> the columns k = k' * world +
    rank, contiguous.  This is how the inner dimension of a matrix product is dealt to the provers
    of the sharded ``prove_matmul``."""
    if K % world:
        raise ValueError("the number of provers must divide the inner dimension")
    return np.ascontiguousarray(np.asarray(t).reshape(-1, K)[:, rank::world])


def gather_partials(part, dist=None):
    """All-gather of one small per-rank buffer into [world, n], in rank order.  A CUDA torch tensor is
    gathered in place on the GPU (NCCL over NVLink); a numpy uint32 array goes through the process
    group's CPU path (gloo)."""
    if dist is None or dist.get_world_size() == 1:
        return part.reshape(1, -1)
    import torch
    world = dist.get_world_size()
    if isinstance(part, torch.Tensor):
        out = torch.empty((world, part.numel()), dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(out, part.reshape(-1))
        return out
    flat = np.ascontiguousarray(part, dtype=np.uint32).reshape(-1)
    mine = torch.from_numpy(flat.astype(np.int64))
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    return np.stack([p.numpy().astype(np.uint32) for p in parts])


def prove_matmul_sharded(ctx, d_A_shard, d_B_shard, L: int, N: int, M: int, K: int, u, v, claim: int, dist=None):
    """``prove_matmul`` with the inner dimension dealt to the ranks by residue class (this rank holds
    ``shard_columns(A, K, rank, world)`` as an Fr tensor on its GPU).  Each rank folds its shard and
    runs the local rounds, ONE all-gather of a few hundred bytes per rank crosses NVLink, and every
    rank finishes the proof (partial sums added mod r on the device, last log2(world) rounds, round
    checks).  Returns what ``host.prove_matmul`` returns, bit-identical to the unsharded proof."""
    import torch
    from . import host
    world = 1 if dist is None else dist.get_world_size()
    if world & (world - 1) or K % world:
        raise ValueError("the number of ranks must be a power of two that divides the inner dimension")
    lp = world.bit_length() - 1
    k_local = K // world
    n_el = host.matmul_partial_elems(L, k_local)
    device = torch.device("cuda", torch.cuda.current_device())
    # torch runs under the library's own stream here: the collective is ordered after the partial
    # proof and before the finish on the device, without a host synchronisation on either side
    with torch.cuda.stream(library_stream(ctx)):
        part = torch.empty(n_el * 8, dtype=torch.int32, device=device)
        host.prove_matmul_partial(ctx, d_A_shard, d_B_shard, L, N, M, k_local, u, list(v)[lp:], part.data_ptr())
        gathered = gather_partials(part, dist)
        return host.prove_matmul_finish(ctx, gathered.data_ptr(), world, L, N, M, K, u, v, claim)


def max_over_ranks(value: float, dist=None, device: str = "cpu") -> float:
    """Maximum of a per-rank timing (the number multi-GPU throughput is computed from)."""
    if dist is None or dist.get_world_size() == 1:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
