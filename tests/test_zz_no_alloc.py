"""The allocation-free commitment entry point must agree, byte for byte, with the regular one (and both
with the C restatement of the reference's commit).

Some embedders cannot allocate device memory at the moment they commit (a framework that owns all
GPU memory through its own pool, or a latency-critical loop where cudaMalloc's implicit
synchronisation is unacceptable).  ``grape_commit_i32_static`` keeps its partial sums in a fixed
array inside the library instead of the context's arena.  This file is collected last so that a
run stopping at the first failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_commit(g, ctx, table, d_scalars, size, wd, max_bits, d_out):
    lib = ctx.lib
    st = C.c_uint32(99)
    rc = lib.grape_commit_i32_static(C.c_void_p(lib.grape_table_data(table.handle)), table.n_gens,
                                     table.window_bits, table.n_windows, C.c_void_p(d_scalars.ptr), size, wd,
                                     max_bits, C.c_void_p(d_out.ptr), C.c_void_p(ctx.stream), C.byref(st))
    return rc, st.value


@pytest.mark.parametrize("window_bits,rows,wd", [(8, 7, 200), (16, 300, 64)])
def test_static_commit_matches_arena_commit_twice(window_bits, rows, wd):
    import grape_b200 as g
    from grape_b200 import workloads as wl
    ctx = g.Context(0)
    lib = ctx.lib
    lib.grape_static_scratch_bytes.restype = C.c_uint64
    lib.grape_static_error.restype = C.c_char_p
    assert lib.grape_static_scratch_bytes() == 65536 * 128
    gens = wl.make_generators(ctx, max(wd, 64), seed=21)
    table = g.GeneratorTable(ctx, gens, window_bits, 1)
    from oracle import cport
    ctable = cport.table_build(gens)
    rng = np.random.default_rng(window_bits)
    want_out, got_out = ctx.alloc(rows * 96), ctx.alloc(rows * 96)
    for call in range(2):  # two calls in a row share the static array
        s = rng.integers(-2**15, 2**15, size=rows * wd).astype(np.int32)
        if call == 1:
            s[: wd] = 0  # a row that commits to infinity, after a call that left other data behind
        d = ctx.upload(s)
        g.commit_i32(ctx, table, d, s.size, wd, want_out, max_bits=16)
        want = ctx.download(want_out, rows * 96)
        rc, status = _static_commit(g, ctx, table, d, s.size, wd, 16, got_out)
        assert rc == 0, lib.grape_static_error()
        assert status == 0
        got = ctx.download(got_out, rows * 96)
        assert got.tobytes() == want.tobytes()
        assert got.tobytes() == cport.commit_i32(s, wd, ctable[:, :wd].copy()).tobytes()   # and the reference's rows
    # sizes beyond the fixed scratch are refused, not truncated
    big_rows = 65537
    rc, _ = _static_commit(g, ctx, table, want_out, big_rows * wd, wd, 16, got_out)
    assert rc == 5  # GRAPE_ERR_LIMIT
    assert b"limit" in lib.grape_static_error()
    # a table geometry that grape_table_create would refuse is refused here too
    rc = lib.grape_commit_i32_static(C.c_void_p(lib.grape_table_data(table.handle)), table.n_gens, 16, 17,
                                     C.c_void_p(want_out.ptr), rows * wd, wd, 16, C.c_void_p(got_out.ptr),
                                     C.c_void_p(ctx.stream), None)
    assert rc == 1 and b"geometry" in lib.grape_static_error()
    table.close()
    ctx.close()
