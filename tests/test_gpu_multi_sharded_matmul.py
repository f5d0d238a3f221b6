"""The sharded matrix-product sumcheck over real ranks: two processes, one GPU each, NCCL all-gather.
Skipped on a box with a single GPU (the single-GPU emulation in test_gpu_sumcheck.py and the gloo
test cover the same logic there)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import random
    import torch
    import torch.distributed as dist
    import grape_b200 as g
    from grape_b200 import host, parallel
    from oracle import bn254, protocols as pr
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        ctx = g.Context(rank)
        R = bn254.R
        rnd = random.Random(41)
        L, N, M, K = 2, 4, 8, 24
        A = [rnd.randrange(-2**15, 2**15) % R for _ in range(L * N * K)]
        B = [rnd.randrange(-2**15, 2**15) % R for _ in range(L * M * K)]
        u = [rnd.randrange(R) for _ in range(pr.log2ceil(L * N * M))]
        v = [rnd.randrange(R) for _ in range(pr.log2ceil(L * K))]
        a_ = pr.partial_eval(list(A), len(A), u, N, pr.log2ceil(M), K)
        b_ = pr.partial_eval(list(B), len(B), u, M, 0, K)
        lL, u_end = pr.log2ceil(L), pr.log2ceil(L * N * M)
        w = pr.eq_weights(u[u_end - lL:u_end], lL, L)
        claim = sum(w[l] * a_[l * K + k] * b_[l * K + k] for l in range(L) for k in range(K)) % R
        want = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
        As = np.ascontiguousarray(host.encode_field(A).reshape(-1, K, 8)[:, rank::world, :])
        Bs = np.ascontiguousarray(host.encode_field(B).reshape(-1, K, 8)[:, rank::world, :])
        got = parallel.prove_matmul_sharded(ctx, ctx.upload(As), ctx.upload(Bs), L, N, M, K, u, v, claim, dist)
        ok = got[:3] == want[:3] and got[3] == [list(p) + [0] * (4 - len(p)) for p in want[3]]
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_prove_matmul_over_nccl():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    mctx = mp.get_context("spawn")
    q = mctx.Queue()
    procs = [mctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
