"""Parity of the Hyrax row commitments (table build + MSM) against the oracle's group arithmetic."""
import random

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
R = bn254.R


@pytest.fixture(scope="module")
def gens64():
    return bn254.make_generators(64, seed=0xC1)


def _commit(gctx, table, scalars, wd, max_bits):
    import grape_b200 as g
    arr = np.array(scalars, dtype=np.int32)
    d = gctx.upload(arr)
    rows = arr.size // wd
    out = gctx.alloc(max(rows, 1) * 96)
    g.commit_i32(gctx, table, d, arr.size, wd, out, max_bits=max_bits)
    raw = gctx.download(out, rows * 96).reshape(rows, 24)
    assert gctx.status() == 0
    return raw


@pytest.mark.parametrize("window_bits,n_windows", [(8, 1), (8, 4), (16, 1), (16, 2), (12, 1), (13, 3), (7, 2), (10, 1)])
def test_commit_i32_full_range(gctx, gens64, window_bits, n_windows):
    import grape_b200 as g
    rng = random.Random(window_bits * 10 + n_windows)
    wd, rows = 64, 9
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), window_bits, n_windows)
    s = [rng.randrange(-2**31, 2**31) for _ in range(rows * wd)]
    s[:8] = [0, 1, -1, 2**31 - 1, -2**31, 128, -128, 32768]
    s[wd:2 * wd] = [0] * wd  # an all-zero row commits to infinity
    raw = _commit(gctx, table, s, wd, 32)
    want = pr.commit_rows(s, wd, gens64)
    assert g.decode_jacobian(raw) == want
    assert raw.tobytes() == b"".join(bn254.jacobian_to_bytes(p) for p in want)  # canonical Z = 1 records
    table.close()


@pytest.mark.parametrize("window_bits", [8, 16])
def test_commit_i16_range_with_hint(gctx, gens64, window_bits):
    import grape_b200 as g
    rng = random.Random(7)
    wd, rows = 48, 5  # fewer scalars per row than generators in the table
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), window_bits, 1)
    s = [rng.randrange(-2**15, 2**15) for _ in range(rows * wd)]
    s[:4] = [-32768, 32767, 0, -1]
    raw = _commit(gctx, table, s, wd, 16)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, wd, gens64)
    table.close()


def test_commit_many_chunks_single_row(gctx):
    """One long row is split over many blocks and reduced through scratch memory."""
    import grape_b200 as g
    gens = bn254.make_generators(700, seed=3)
    rng = random.Random(1)
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens), 8, 1)
    s = [rng.randrange(-2**31, 2**31) for _ in range(700)]
    raw = _commit(gctx, table, s, 700, 32)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, 700, gens)
    table.close()


def test_commit_degenerate_generators(gctx):
    """Equal, opposite and infinite generators exercise the doubling / cancellation branches."""
    import grape_b200 as g
    G = bn254.G1_GEN
    g5 = bn254.scalar_mul(5, G)
    gens = [G, G, bn254.neg(G), None, g5, g5, bn254.neg(g5), G] * 4
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens), 8, 1)
    rows = [[1] * 32, [3, -3, 0, 9] * 8, [1, 0, 1, 0, 0, 0, 0, 0] * 4, [2, -1, 1, 5, 0, 0, 0, -2] * 4]
    s = [v for r in rows for v in r]
    raw = _commit(gctx, table, s, 32, 32)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, 32, gens)
    table.close()


@pytest.mark.parametrize("window_bits,n_windows", [(8, 1), (16, 1), (8, 32), (13, 1), (11, 2), (5, 1)])
def test_commit_fr(gctx, gens64, window_bits, n_windows):
    import grape_b200 as g
    rng = random.Random(99)
    wd, rows = 64, 4
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), window_bits, n_windows)
    s = [rng.randrange(R) for _ in range(rows * wd)]
    s[:5] = [0, 1, R - 1, (1 << 253), 0x80]
    s[wd:wd + 8] = [3, 0, 0, 7, 2**16, 2**32 - 1, 5, 0]  # small multiplicities
    d = gctx.fr_upload(s)
    out = gctx.alloc(rows * 96)
    g.commit_fr(gctx, table, d, rows * wd, wd, out)
    raw = gctx.download(out, rows * 96).reshape(rows, 24)
    assert g.decode_jacobian(raw) == pr.commit_rows(s, wd, gens64)
    assert gctx.fr_download(d, 5) == s[:5]  # scalars are left untouched
    table.close()


def test_commit_host_buffers(gctx, gens64):
    import grape_b200 as g
    rng = np.random.default_rng(2)
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), 8, 1)
    s = rng.integers(-2**15, 2**15, size=64 * 7).astype(np.int32)
    raw = g.commit_i32_host(gctx, table, s, 64, max_bits=16)
    assert g.decode_jacobian(raw) == pr.commit_rows([int(v) for v in s], 64, gens64)
    table.close()


@pytest.mark.parametrize("rows", [4096, 4099, 5000])
def test_commit_host_buffers_sliced_pipeline(gctx, gens64, rows):
    """From 4096 rows on, the host-buffer entry point copies and commits in uneven row slices on two
    streams; every row must come out as the device-resident entry point computes it."""
    import grape_b200 as g
    rng = np.random.default_rng(rows)
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), 8, 1)
    s = rng.integers(-2**15, 2**15, size=rows * 64).astype(np.int32)
    raw = g.commit_i32_host(gctx, table, s, 64, max_bits=16)
    d_out = gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, gctx.upload(s), rows * 64, 64, d_out, max_bits=16)
    assert np.array_equal(raw, gctx.download(d_out, rows * 96).reshape(rows, 24))
    # spot-check rows at the slice boundaries against the oracle
    for r in {0, rows // 32 - 1, rows // 32, rows * 4 // 32, rows * 11 // 32, rows * 21 // 32, rows - 1}:
        assert g.decode_jacobian(raw[r:r + 1]) == pr.commit_rows([int(v) for v in s[r * 64:(r + 1) * 64]], 64, gens64)
    table.close()


def test_commit_host_buffers_page_locked_read_in_place(gctx, gens64):
    """Page-locked scalars are read by the kernel where they lie (no staging copy); pageable ones are staged:
    both must give the records of the device-resident entry point, and the address helper refuses pageable memory."""
    import grape_b200 as g
    rows = 4500
    rng = np.random.default_rng(77)
    pageable = rng.integers(-2**15, 2**15, size=rows * 64).astype(np.int32)
    pinned = gctx.pinned_array((rows * 64,), np.int32)
    pinned[...] = pageable
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), 16, 1)
    a = g.commit_i32_host(gctx, table, pinned, 64, max_bits=16)
    b = g.commit_i32_host(gctx, table, pageable, 64, max_bits=16)
    d_out = gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, gctx.host_device_pointer(pinned), rows * 64, 64, d_out, max_bits=16)
    c = gctx.download(d_out, rows * 96).reshape(rows, 24)
    assert np.array_equal(a, b) and np.array_equal(a, c)
    assert g.decode_jacobian(a[:3]) == pr.commit_rows([int(v) for v in pageable[:3 * 64]], 64, gens64)
    with pytest.raises(g.GrapeError):
        gctx.host_device_pointer(pageable)
    table.close()


def test_commit_rejects_bad_shapes(gctx, gens64):
    import grape_b200 as g
    table = g.GeneratorTable(gctx, g.encode_jacobian(gens64), 8, 1)
    d = gctx.alloc(4 * 130)
    out = gctx.alloc(96 * 4)
    with pytest.raises(g.GrapeError):
        g.commit_i32(gctx, table, d, 130, 65, out)  # more scalars per row than generators
    with pytest.raises(g.GrapeError):
        g.commit_i32(gctx, table, d, 130, 64, out)  # size not a multiple of the row length
    table.close()
