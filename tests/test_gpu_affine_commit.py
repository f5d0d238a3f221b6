"""The commitment kernel with affine accumulators and shared inversions against the oracle and against the
extended-coordinate kernel: same group elements, byte for byte, whatever the split into slots and chunks."""
import random

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
R = bn254.R


def _commit_i32(gctx, table, arr, wd, max_bits):
    import grape_b200 as g
    rows = arr.size // wd
    out = gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, gctx.upload(arr), arr.size, wd, out, max_bits=max_bits)
    raw = gctx.download(out, rows * 96).reshape(rows, 24)
    assert gctx.status() == 0
    return raw


@pytest.mark.parametrize("window_bits,n_windows,slots,chunks", [(8, 1, 8, 1), (16, 1, 16, 2), (13, 2, 64, 1), (7, 1, 24, 3)])
def test_affine_commit_i32_matches_oracle(gctx, window_bits, n_windows, slots, chunks):
    import grape_b200 as g
    gens = bn254.make_generators(100, seed=0xAF)
    rng = random.Random(slots)
    wd, rows = 100, 21  # neither a multiple of the lane count nor of the slots per lane
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens), window_bits, n_windows)
    s = [rng.randrange(-2**31, 2**31) for _ in range(rows * wd)]
    s[:8] = [0, 1, -1, 2**31 - 1, -2**31, 128, -128, 32768]
    s[wd:2 * wd] = [0] * wd  # a row that commits to infinity
    arr = np.array(s, dtype=np.int32)
    try:
        gctx.set_affine_commit(2, slots, chunks)
        raw = _commit_i32(gctx, table, arr, wd, 32)
    finally:
        gctx.set_affine_commit(-1)
    want = pr.commit_rows(s, wd, gens)
    assert g.decode_jacobian(raw) == want
    assert raw.tobytes() == b"".join(bn254.jacobian_to_bytes(p) for p in want)
    table.close()


def test_affine_commit_degenerate_generators(gctx):
    """Equal, opposite and infinite generators drive the tangent, cancellation and copy cases of the affine
    addition, in runs (an accumulator that went back to infinity is filled again)."""
    import grape_b200 as g
    G = bn254.G1_GEN
    g5 = bn254.scalar_mul(5, G)
    gens = ([G] * 32 + [G] * 32 + [bn254.neg(G)] * 32 + [None] * 32 + [g5] * 32 + [g5] * 32 + [G] * 32 + [G] * 32)
    wd = len(gens)
    rng = random.Random(5)
    rows = [[1] * wd, [3, -3, 0, 9] * (wd // 4), [rng.randrange(-3, 4) for _ in range(wd)],
            [rng.randrange(-2, 3) for _ in range(wd)], [2] * 64 + [4] * 32 + [7] * 32 + [-1] * 64 + [5] * 64]
    rows += [[rng.randrange(-1, 2) for _ in range(wd)] for _ in range(12)]
    s = [v for r in rows for v in r]
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens), 8, 1)
    arr = np.array(s, dtype=np.int32)
    try:
        gctx.set_affine_commit(2, 8, 1)
        raw = _commit_i32(gctx, table, arr, wd, 32)
    finally:
        gctx.set_affine_commit(-1)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, wd, gens)
    table.close()


@pytest.mark.parametrize("window_bits,n_windows,slots,chunks", [(13, 1, 32, 1), (8, 4, 16, 2), (16, 1, 40, 1)])
def test_affine_commit_fr_matches_oracle(gctx, window_bits, n_windows, slots, chunks):
    import grape_b200 as g
    gens = bn254.make_generators(64, seed=0xC1)
    rng = random.Random(99 + slots)
    wd, rows = 64, 5
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens), window_bits, n_windows)
    s = [rng.randrange(R) for _ in range(rows * wd)]
    s[:5] = [0, 1, R - 1, (1 << 253), 0x80]
    s[wd:wd + 8] = [3, 0, 0, 7, 2**16, 2**32 - 1, 5, 0]
    d = gctx.fr_upload(s)
    out = gctx.alloc(rows * 96)
    try:
        gctx.set_affine_commit(2, slots, chunks)
        g.commit_fr(gctx, table, d, rows * wd, wd, out)
    finally:
        gctx.set_affine_commit(-1)
    raw = gctx.download(out, rows * 96).reshape(rows, 24)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, wd, gens)
    table.close()


@pytest.mark.parametrize("rows,wd,slots,chunks", [(3000, 512, 0, 0), (777, 1000, 64, 0), (4096, 256, 56, 2)])
def test_affine_commit_equals_extended_kernel(gctx, rows, wd, slots, chunks):
    """At sizes the oracle cannot walk: both kernels must write the same bytes (int16 scalars and 16-bit
    windows as in the layer commitments, then Fr scalars on 13-bit windows as in the lookups)."""
    import grape_b200 as g
    from grape_b200 import workloads as wl
    gens = wl.make_generators(gctx, wd, seed=11)
    rng = np.random.default_rng(rows)
    for window_bits, fr in ((16, False), (13, True)):
        table = g.GeneratorTable(gctx, gens, window_bits, 1)
        n = rows * wd if not fr else (rows // 8) * wd
        s = rng.integers(-2**15, 2**15, size=n).astype(np.int32)
        s[::97] = 0
        d_i = gctx.upload(s)
        if fr:
            d = gctx.alloc(n * 32)
            gctx.fr_from_i32(d_i, n, d)   # negative values become full-width residues
        outs = []
        for mode in ((0, 0, 0), (2, slots, chunks)):
            gctx.set_affine_commit(*mode)
            try:
                o = gctx.alloc((n // wd) * 96)
                if fr:
                    g.commit_fr(gctx, table, d, n, wd, o)
                else:
                    g.commit_i32(gctx, table, d_i, n, wd, o, max_bits=16)
                outs.append(gctx.download(o, (n // wd) * 96).tobytes())
            finally:
                gctx.set_affine_commit(-1)
        assert outs[0] == outs[1]
        assert gctx.status() == 0
        table.close()
