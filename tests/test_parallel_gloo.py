"""Row sharding across ranks with two CPU processes over gloo (the N > 1 path without GPUs): blocks
are contiguous, uneven row counts are handled, gathered records come back in row order, and timing
is the maximum over ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grape_b200 import parallel


def test_row_block_partition():
    for rows in (0, 1, 7, 8, 49408):
        for world in (1, 2, 3, 8):
            blocks = [parallel.row_block(rows, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == rows
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in blocks]
            assert max(sizes) - min(sizes) <= 1


def _fake_commit(block: np.ndarray, wd: int) -> np.ndarray:
    """Stand-in for the GPU commit: a deterministic 24-word record per row."""
    rows = block.reshape(-1, wd).astype(np.int64)
    rec = np.zeros((rows.shape[0], 24), dtype=np.uint32)
    for k in range(24):
        rec[:, k] = ((rows * (k + 3)).sum(axis=1) & 0xFFFFFFFF).astype(np.uint32)
    return rec


def _worker(rank, world, port, rows, wd, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(3)
    scalars = rng.integers(-2**15, 2**15, size=rows * wd).astype(np.int32)
    got = parallel.commit_rows_sharded(scalars, wd, lambda s: _fake_commit(s, wd), dist)
    t = parallel.max_over_ranks(10.0 + rank, dist)
    q.put((rank, got.tobytes(), t))
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [7, 8])
def test_two_rank_row_sharding_over_gloo(rows):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    wd, world = 5, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, rows, wd, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rng = np.random.default_rng(3)
    scalars = rng.integers(-2**15, 2**15, size=rows * wd).astype(np.int32)
    want = _fake_commit(scalars, wd).tobytes()
    for rank, blob, t in results:
        assert blob == want
        assert t == 11.0


# ---- the matrix-product sumcheck split over two provers ------------------------------------------
def _matmul_case():
    import random
    from oracle import bn254, protocols as pr
    R = bn254.R
    rnd = random.Random(17)
    L, N, M, K = 2, 3, 4, 12
    A = [rnd.randrange(-99, 99) % R for _ in range(L * N * K)]
    B = [rnd.randrange(-99, 99) % R for _ in range(L * M * K)]
    u = [rnd.randrange(R) for _ in range(pr.log2ceil(L * N * M))]
    v = [rnd.randrange(R) for _ in range(pr.log2ceil(L * K))]
    a_ = pr.partial_eval(list(A), len(A), u, N, pr.log2ceil(M), K)
    b_ = pr.partial_eval(list(B), len(B), u, M, 0, K)
    lL, u_end = pr.log2ceil(L), pr.log2ceil(L * N * M)
    w = pr.eq_weights(u[u_end - lL:u_end], lL, L)
    claim = sum(w[l] * a_[l * K + k] * b_[l * K + k] for l in range(L) for k in range(K)) % R
    return L, N, M, K, A, B, u, v, claim


def _sumcheck_worker(rank, world, port, q):
    from oracle import bn254, protocols as pr
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L, N, M, K, A, B, u, v, claim = _matmul_case()
    # this rank's residue-class shard, cut with the library's own helper (object arrays keep the integers exact)
    As = parallel.shard_columns(np.array(A, dtype=object), K, rank, world).reshape(-1).tolist()
    Bs = parallel.shard_columns(np.array(B, dtype=object), K, rank, world).reshape(-1).tolist()
    lp = world.bit_length() - 1
    sums, a, b = pr.prove_matmul_partial(As, Bs, L, N, M, K // world, u, v[lp:])
    flat = [x for q3 in sums for x in q3] + [a, b]
    part = np.frombuffer(bn254.fr_vec_to_bytes(flat), dtype=np.uint32)
    gathered = parallel.gather_partials(part, dist)           # the one exchange of the sharded proof
    assert gathered.shape == (world, len(flat) * 8)
    parts = []
    for r in range(world):
        vals = bn254.fr_vec_from_bytes(gathered[r].tobytes())
        parts.append(([vals[3 * i:3 * i + 3] for i in range(len(sums))], vals[-2], vals[-1]))
    got = pr.prove_matmul_finish(parts, L, N, M, K, u, v, claim)
    q.put((rank, got))
    dist.destroy_process_group()


def test_two_rank_sharded_matmul_sumcheck_over_gloo():
    from oracle import protocols as pr
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sumcheck_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    L, N, M, K, A, B, u, v, claim = _matmul_case()
    want = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
    for rank, got in results:
        assert got == want        # every rank ends with the unsharded proof, transcript included
