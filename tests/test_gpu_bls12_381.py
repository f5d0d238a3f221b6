"""BLS12-381 instantiation of the commitment path against the Python oracle (oracle/bls12_381.py).

The reference never compiles this curve, so parity here is against the oracle only: field
arithmetic on 12 x 32-bit limbs (Fp) and 8 limbs (Fr), the generator table, and row commitments of
int32 and Fr scalars for several window widths, with the special cases of the group law
(zero scalars, repeated generators, a generator at infinity, opposite terms cancelling).
"""
import ctypes as C
import random

import numpy as np
import pytest

from oracle import bls12_381 as bls

pytestmark = pytest.mark.gpu


def _enc(values, mod, nbytes, to_bytes):
    return np.frombuffer(b"".join(to_bytes(v) for v in values), dtype=np.uint32).reshape(len(values), nbytes // 4).copy()


def _enc_fp(vals):
    return _enc(vals, bls.P, 48, bls.fp_to_bytes)


def _enc_fr(vals):
    return _enc(vals, bls.R, 32, bls.fr_to_bytes)


def _enc_jac(points):
    return np.frombuffer(b"".join(bls.jacobian_to_bytes(p) for p in points), dtype=np.uint32).reshape(len(points), 36).copy()


def _dec_jac(arr):
    return bls.jacobian_vec_from_bytes(np.ascontiguousarray(arr, dtype=np.uint32).tobytes())


@pytest.mark.parametrize("field", [0, 1])
def test_field_binary_matches_integers(gctx, field):
    mod = bls.R if field == 0 else bls.P
    nbytes = 32 if field == 0 else 48
    to_b = bls.fr_to_bytes if field == 0 else bls.fp_to_bytes
    from_b = bls.fr_from_bytes if field == 0 else bls.fp_from_bytes
    rnd = random.Random(381 + field)
    a = [0, 1, mod - 1, mod - 1, mod - 2, 2, (mod - 1) // 2, (mod + 1) // 2] + [rnd.randrange(mod) for _ in range(500)]
    b = [0, mod - 1, mod - 1, 1, mod - 2, (mod + 1) // 2, (mod - 1) // 2, (mod + 1) // 2] + [rnd.randrange(mod) for _ in range(500)]
    # raw Montgomery residues at the top of the range as well: x * R mod m == m - 1
    da, db = gctx.upload(_enc(a, mod, nbytes, to_b)), gctx.upload(_enc(b, mod, nbytes, to_b))
    out = gctx.alloc(len(a) * nbytes)
    for op, fn in ((0, lambda x, y: (x + y) % mod), (1, lambda x, y: (x - y) % mod), (2, lambda x, y: x * y % mod)):
        gctx._check(gctx.lib.grape_bls12_381_field_binary(gctx.handle, field, op, da.ptr, db.ptr, out.ptr, len(a)))
        raw = gctx.download(out, len(a) * nbytes).tobytes()
        got = [from_b(raw[i * nbytes:(i + 1) * nbytes]) for i in range(len(a))]
        assert got == [fn(x, y) for x, y in zip(a, b)], f"field {field} op {op}"
        # stored values are canonical residues
        assert all(int.from_bytes(raw[i * nbytes:(i + 1) * nbytes], "little") < mod for i in range(len(a)))


def test_fr_from_i32(gctx):
    vals = np.array([0, 1, -1, 2**31 - 1, -2**31, 65536, -32768, 12345], dtype=np.int32)
    out = gctx.alloc(len(vals) * 32)
    gctx._check(gctx.lib.grape_bls12_381_fr_from_i32(gctx.handle, gctx.upload(vals).ptr, out.ptr, len(vals)))
    raw = gctx.download(out, len(vals) * 32).tobytes()
    assert [bls.fr_from_bytes(raw[i * 32:(i + 1) * 32]) for i in range(len(vals))] == [int(v) % bls.R for v in vals]


def _gens(n, seed):
    rnd = random.Random(seed)
    return [bls.scalar_mul(rnd.randrange(1, bls.R), bls.G1_GEN) for _ in range(n)]


@pytest.mark.parametrize("window_bits,n_windows,max_bits", [(8, 1, 32), (16, 1, 16), (13, 1, 16), (8, 2, 32), (5, 1, 17)])
def test_commit_i32_matches_oracle(gctx, window_bits, n_windows, max_bits):
    from grape_b200 import host as g
    wd, rows = 16, 6
    gens = _gens(wd, 11)
    gens[3] = gens[2]            # repeated generator: equal scalars hit the doubling branch in the warp tree
    gens[7] = None               # a generator at infinity
    gens[9] = bls.neg(gens[8])   # opposite points: equal scalars cancel
    rnd = random.Random(window_bits * 100 + max_bits)
    lim = 1 << (max_bits - 1)
    t = np.array([rnd.randrange(-lim + 1, lim) for _ in range(rows * wd)], dtype=np.int64)
    t[0:wd] = 0                                   # an all-zero row commits to infinity
    t[wd + 2] = t[wd + 3] = 77                    # same scalar on the repeated generator
    t[2 * wd + 8] = t[2 * wd + 9] = -123          # cancels on the opposite pair
    t[3 * wd:3 * wd + 4] = [lim - 1, -(lim - 1), 1, -1]
    t = t.astype(np.int32)
    table = g.GeneratorTable(gctx, _enc_jac(gens), window_bits, n_windows, curve="bls12_381")
    assert gctx.lib.grape_table_curve(table.handle) == 1
    assert table.nbytes == (1 << (window_bits - 1)) * n_windows * wd * 96
    out = gctx.alloc(rows * 144)
    g.commit_i32(gctx, table, gctx.upload(t), rows * wd, wd, out, max_bits=max_bits)
    got = _dec_jac(gctx.download(out, rows * 144))
    want = bls.commit_rows([int(x) for x in t], wd, gens)
    assert got == want
    # the affine-accumulator kernel on the 12-limb field: same records
    try:
        gctx.set_affine_commit(2, 4, 1)
        out2 = gctx.alloc(rows * 144)
        g.commit_i32(gctx, table, gctx.upload(t), rows * wd, wd, out2, max_bits=max_bits)
        assert _dec_jac(gctx.download(out2, rows * 144)) == want
    finally:
        gctx.set_affine_commit(-1)
    assert got[0] is None
    # the records are canonical: Z is the Montgomery one (or zero for infinity)
    raw = gctx.download(out, rows * 144).tobytes()
    assert raw[144 + 96:144 + 144] == bls.fp_to_bytes(1)
    # the host-buffer entry point gives the same records
    host_out = g.commit_i32_host(gctx, table, t, wd, max_bits=max_bits)
    assert host_out.shape == (rows, 36) and _dec_jac(host_out) == want
    table.close()


@pytest.mark.parametrize("window_bits", [8, 16, 5, 11])
def test_commit_fr_matches_oracle(gctx, window_bits):
    from grape_b200 import host as g
    wd, rows = 8, 3
    gens = _gens(wd, 23)
    rnd = random.Random(window_bits)
    s = [rnd.randrange(bls.R) for _ in range(rows * wd)]
    s[0], s[1], s[2], s[3] = 0, bls.R - 1, 1, (bls.R - 1) // 2
    s[8], s[9] = (1 << 254) + 12345, (1 << 255) % bls.R
    table = g.GeneratorTable(gctx, _enc_jac(gens), window_bits, 1, curve="bls12_381")
    out = gctx.alloc(rows * 144)
    g.commit_fr(gctx, table, gctx.upload(_enc_fr(s)), rows * wd, wd, out)
    got = _dec_jac(gctx.download(out, rows * 144))
    assert got == bls.commit_rows(s, wd, gens)
    table.close()


def test_long_rows_split_over_warps(gctx):
    """Few long rows: each row is split into chunks handled by different warps and re-assembled."""
    from grape_b200 import host as g
    wd, rows = 256, 2
    base = _gens(8, 5)
    gens = [base[i % 8] if i < 8 else bls.add(base[i % 8], base[(i // 8) % 8]) for i in range(wd)]
    rnd = random.Random(9)
    t = np.array([rnd.randrange(-2**15, 2**15) for _ in range(rows * wd)], dtype=np.int32)
    table = g.GeneratorTable(gctx, _enc_jac(gens), 8, 1, curve="bls12_381")
    out = gctx.alloc(rows * 144)
    g.commit_i32(gctx, table, gctx.upload(t), rows * wd, wd, out, max_bits=16)
    assert _dec_jac(gctx.download(out, rows * 144)) == bls.commit_rows([int(x) for x in t], wd, gens)
    table.close()


def test_bn254_only_entry_points_reject_a_bls_table(gctx):
    from grape_b200 import host as g
    table = g.GeneratorTable(gctx, _enc_jac(_gens(16, 1)), 8, 1, curve="bls12_381")
    with pytest.raises(Exception):
        g.hyrax_open(gctx, table, gctx.alloc(16 * 32), 16, 1, 1, [0, 0, 0, 0], 1, np.zeros(24, dtype=np.uint32))
    table.close()


def test_synthetic_generators_are_multiples_of_the_standard_generator(gctx):
    from grape_b200 import workloads as wl
    gens = wl.make_generators_bls12_381(gctx, 5, seed=77)
    gctx.seed(77)
    rho = gctx.random_fr(5).tobytes()
    want = [bls.scalar_mul(bls.fr_from_bytes(rho[i * 32:(i + 1) * 32]), bls.G1_GEN) for i in range(5)]
    assert _dec_jac(gens) == want


def test_host_buffer_pipeline_in_slices(gctx):
    """From 4096 rows on the host-buffer entry point works in row slices on two streams; on this curve
    the records are 144 bytes.  Every row must equal the device-resident result."""
    from grape_b200 import host as g
    wd, rows = 16, 4100
    gens = _gens(wd, 31)
    rng = np.random.default_rng(4100)
    t = rng.integers(-2**15, 2**15, size=rows * wd).astype(np.int32)
    table = g.GeneratorTable(gctx, _enc_jac(gens), 8, 1, curve="bls12_381")
    host_out = g.commit_i32_host(gctx, table, t, wd, max_bits=16)
    d_out = gctx.alloc(rows * 144)
    g.commit_i32(gctx, table, gctx.upload(t), rows * wd, wd, d_out, max_bits=16)
    assert np.array_equal(host_out, gctx.download(d_out, rows * 144).reshape(rows, 36))
    for r in (0, 127, 128, 4099):
        assert _dec_jac(host_out[r:r + 1]) == bls.commit_rows([int(x) for x in t[r * wd:(r + 1) * wd]], wd, gens)
    table.close()
