"""Bit-exact parity of the Fr / Fp device arithmetic against the big-integer oracle."""
import random

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu

R, P = bn254.R, bn254.P


def _edge_values(mod, rng, n):
    vals = [0, 1, 2, mod - 1, mod - 2, (1 << 253), (1 << 253) + 1, mod >> 1, 0xFFFFFFFF, 1 << 32, (1 << 224) - 1]
    vals += [rng.randrange(mod) for _ in range(n - len(vals))]
    return vals


@pytest.mark.parametrize("field", ["fr", "fp"])
@pytest.mark.parametrize("op", ["add", "sub", "mul"])
def test_binary_ops(gctx, field, op):
    import grape_b200 as g
    rng = random.Random(11)
    mod = R if field == "fr" else P
    n = 4099
    a = _edge_values(mod, rng, n)
    b = list(reversed(_edge_values(mod, rng, n)))
    da, db = gctx.upload(g.encode_field(a, mod)), gctx.upload(g.encode_field(b, mod))
    out = gctx.alloc(n * 32)
    (gctx.fr_binary if field == "fr" else gctx.fp_binary)(op, da, db, out, n)
    got = g.decode_field(gctx.download(out, n * 32), mod)
    f = {"add": lambda x, y: (x + y) % mod, "sub": lambda x, y: (x - y) % mod, "mul": lambda x, y: x * y % mod}[op]
    assert got == [f(x, y) for x, y in zip(a, b)]
    # canonical residues: every output limb vector is < modulus
    raw = gctx.download(out, n * 32).reshape(-1, 8)
    for row in raw[:64]:
        assert int.from_bytes(row.tobytes(), "little") < mod


def test_from_i32_and_mont_roundtrip(gctx):
    import grape_b200 as g
    rng = np.random.default_rng(5)
    x = rng.integers(-2**31, 2**31, size=5000, dtype=np.int64).astype(np.int32)
    x[:6] = [0, 1, -1, 2**31 - 1, -2**31, -32768]
    d = gctx.upload(x)
    out = gctx.alloc(x.size * 32)
    gctx.fr_from_i32(d, x.size, out)
    raw = gctx.download(out, x.size * 32)
    assert raw.tobytes() == bn254.fr_vec_to_bytes([int(v) for v in x])
    # leaving and re-entering Montgomery form
    gctx.fr_from_mont(out, x.size)
    std = gctx.download(out, x.size * 32).reshape(-1, 8)
    assert [int.from_bytes(r.tobytes(), "little") for r in std] == [int(v) % R for v in x]
    gctx.fr_to_mont(out, x.size)
    assert gctx.download(out, x.size * 32).tobytes() == raw.tobytes()
    u = rng.integers(0, 2**32, size=100, dtype=np.uint64).astype(np.uint32)
    du = gctx.upload(u)
    gctx.fr_from_u32(du, u.size, out)
    assert g.decode_field(gctx.download(out, u.size * 32)) == [int(v) for v in u]


@pytest.mark.parametrize("field", [0, 1, 2, 3])
def test_squaring_and_euclid_inverse_agree_with_multiplication(gctx, field):
    """The dedicated squaring equals a*a and the Euclid inversion equals the Fermat ladder, on edge values
    (0, 1, 2, m-1, powers of two, all-ones limbs) and random elements of all four fields."""
    from oracle import bls12_381
    mod = [P, R, bls12_381.P, bls12_381.R][field]
    limbs = 12 if field == 2 else 8
    rng = random.Random(40 + field)
    vals = [0, 1, 2, 3, mod - 1, mod - 2, mod >> 1, (mod >> 1) + 1, 0xFFFFFFFF, 1 << 32, (1 << 64) - 1]
    vals += [(1 << k) % mod for k in range(0, 32 * limbs, 13)]
    vals += [((1 << (32 * limbs)) - 1 - (1 << k)) % mod for k in range(0, 32 * limbs, 29)]
    vals += [rng.randrange(mod) for _ in range(3000)]
    # the kernel takes Montgomery residues: any canonical value is one, so the raw integers are used as given
    raw = b"".join(int(v).to_bytes(4 * limbs, "little") for v in vals)
    d = gctx.upload(np.frombuffer(raw, dtype=np.uint32))
    assert gctx.field_check(field, d, len(vals)) == 0


def test_inverse_sum_rowsum(gctx):
    import grape_b200 as g
    rng = random.Random(3)
    n = 70001
    a = [rng.randrange(R) for _ in range(n)]
    a[5] = 0
    beta = rng.randrange(R)
    a[77] = (-beta) % R  # becomes zero after the shift
    da = gctx.fr_upload(a)
    dbeta = gctx.fr_upload([beta])
    out = gctx.alloc(n * 32)
    gctx.fr_inverse(da, out, n, dbeta)
    got = gctx.fr_download(out, n)
    sample = range(n)   # every element: one product per element checks the inverse
    for i in sample:
        s = (a[i] + beta) % R
        assert got[i] * s % R == (1 if s else 0), i
    # in place, no shift
    gctx.fr_inverse(da, da, n)
    got = gctx.fr_download(da, n)
    for i in sample:
        assert got[i] * a[i] % R == (1 if a[i] else 0), i
        assert a[i] or got[i] == 0
    # sums
    db = gctx.fr_upload(a)
    one = gctx.alloc(32)
    for m in (1, 2, 255, 256, 257, 4097, n):
        gctx.fr_sum(db, m, one)
        assert gctx.fr_download(one, 1)[0] == sum(a[:m]) % R
    rows, dim = 37, 45
    gctx.fr_rowsum(db, out, rows, dim)
    got = gctx.fr_download(out, rows * dim)
    for r in range(rows):
        s = sum(a[r * dim:(r + 1) * dim]) % R
        assert got[r * dim:(r + 1) * dim] == [s] * dim


@pytest.mark.parametrize("other,c,gap", [(1, 8, 1), (3, 11, 1), (2, 6, 5), (1, 64, 300), (4, 13, 33), (1, 1, 7), (5, 2, 1),
                                         (1, 16384, 1), (2, 24576, 1), (1, 8200, 1)])
def test_fold_matches_reference_fold(gctx, other, c, gap):
    rng = random.Random(other * 1000 + c * 10 + gap)
    n = other * c * gap
    t = [rng.randrange(R) for _ in range(n)]
    x = [rng.randrange(R) for _ in range(pr.log2ceil(c) + 2)]
    want = pr.partial_eval(t, n, x, c, 1, gap)
    dt, dx = gctx.fr_upload(t), gctx.fr_upload(x)
    out = gctx.alloc(max(1, other * gap) * 32)
    gctx.fr_fold(dt, n, dx.at(32), c, gap, out)
    assert gctx.fr_download(out, other * gap) == want
    # the same fold straight from int32 data
    ti = [rng.randrange(-2**31, 2**31) for _ in range(n)]
    dti = gctx.upload(np.array(ti, dtype=np.int32))
    gctx.fold_i32(dti, n, dx.at(32), c, gap, out)
    assert gctx.fr_download(out, other * gap) == pr.partial_eval([v % R for v in ti], n, x, c, 1, gap)
