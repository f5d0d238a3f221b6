"""One commitment's rows dealt to two GPUs (Hyrax::commit over row blocks, src/Hyrax.cu:312-333): every
rank commits its contiguous block and one NCCL all-gather on device buffers, issued on the library's
stream, gives every rank all the records.  The gathered records must equal the oracle's rows.  Skipped
on a box with a single GPU (the gloo test of the same partition runs everywhere)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import grape_b200 as g
    from grape_b200 import parallel, workloads as wl
    from oracle import cport
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        ctx = g.Context(rank)
        wd, rows = 256, 96
        gens = wl.make_generators(ctx, wd, 0xC4)            # the same generators on both ranks
        table = g.GeneratorTable(ctx, gens, 16, 1)
        s = np.random.default_rng(4).integers(-(1 << 15), 1 << 15, size=rows * wd).astype(np.int32)
        r0, r1 = parallel.row_block(rows, rank, world)
        block = r1 - r0
        d_block = ctx.upload(s[r0 * wd:r1 * wd])
        d_local, d_all = ctx.alloc(block * 96), ctx.alloc(rows * 96)
        for _ in range(3):                                   # repeated calls reuse the buffers on the stream
            parallel.commit_rows_sharded_device(ctx, table, d_block, block, wd, d_local, d_all, dist, max_bits=16)
        got = ctx.download(d_all, rows * 96).reshape(rows, 24)
        want = cport.commit_i32(s, wd, cport.table_build(gens))
        ok = bool(np.array_equal(got, want))
        # the opening of the same tensor with its rows dealt to the two ranks: same proof as on one GPU
        import random
        from grape_b200 import host
        from oracle import bn254
        rnd = random.Random(9)
        N = wd // 16
        e = [rnd.randrange(bn254.R) for _ in range((rows * wd - 1).bit_length())] if False else None
        rows2 = 64                                            # a power of two for the opening
        e = [rnd.randrange(bn254.R) for _ in range((rows2 * wd - 1).bit_length())]
        cc = rnd.randrange(bn254.R)
        d_fr = ctx.alloc(rows2 * wd * 32)
        ctx.fr_from_i32(ctx.upload(s[:rows2 * wd]), rows2 * wd, d_fr)
        keep = ctx.clone(d_fr, rows2 * wd * 32)
        ctx.seed(1234)
        whole = host.hyrax_open(ctx, table, d_fr, rows2 * wd, N, 1, e, cc, gens[0])
        ctx.seed(1234)
        half = rows2 // world
        shard = parallel.hyrax_open_sharded(ctx, table, keep.at(rank * half * wd * 32), half, rows2, N, e, cc, gens[0], dist)
        ok = ok and shard["result"] == whole["result"] and shard.z_raw.tobytes() == whole.z_raw.tobytes() \
            and shard.com_raw.tobytes() == whole.com_raw.tobytes()
        q.put((rank, ok, ctx.status()))
        table.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_row_sharded_commit_with_nccl_gather():
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
    assert sorted(results) == [(0, True, 0), (1, True, 0)]
