"""CPU oracle, part 1: BN254 (alt_bn128) field and curve arithmetic on Python integers.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the shipped product: only the
tests, the smoke check and the benchmark's CPU-baseline leg may import it, and only as the
checker.

What it restates (paths are relative to the reference project):

* ``include/field/alt_bn128.cuh:11-45``   moduli p (base field) and r (scalar field), the
  Montgomery radix R = 2^256 and the derived constants R mod p/r, R^2 mod p/r.
* ``include/field/mont_t.cuh:453-512``    entering / leaving Montgomery form (value * R mod m).
* ``include/curve/affine_t.cuh:17-75``    affine points, (0, 0) encodes the point at infinity.
* ``include/curve/jacobian_t.cuh``        Jacobian points X|Y|Z, Z = 0 encodes infinity.
* byte layout: a field element is 8 little-endian 32-bit limbs (32 bytes) holding the Montgomery
  residue; an affine point is X|Y (64 bytes); a Jacobian point is X|Y|Z (96 bytes).

Parity status: the arithmetic is mathematically pinned (canonical residues, group elements), the
reference ships no known-answer vectors for it.  The constants below are cross-checked against
the reference's hex literals in ``tests/test_oracle_constants.py``.
"""
from __future__ import annotations

P = 0x30644E72E131A029B85045B68181585D97816A916871CA8D3C208C16D87CFD47  # base field
R = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001  # scalar field
MONT_BITS = 256
MONT_R = 1 << MONT_BITS
CURVE_B = 3  # y^2 = x^3 + 3
G1_GEN = (1, 2)

assert R == 21888242871839275222246405745257275088548364400416034343698204186575808495617
assert P == 21888242871839275222246405745257275088696311157297823662689037894645226208583

MONT_R_INV_P = pow(MONT_R, -1, P)
MONT_R_INV_R = pow(MONT_R, -1, R)


# ----------------------------------------------------------------------------- Montgomery bytes
def to_mont(x: int, mod: int) -> int:
    return (x % mod) * MONT_R % mod


def from_mont(x: int, mod: int) -> int:
    return x * (MONT_R_INV_P if mod == P else MONT_R_INV_R) % mod


def fe_to_bytes(x: int, mod: int) -> bytes:
    """Standard-form integer -> 32-byte little-endian Montgomery residue."""
    return to_mont(x, mod).to_bytes(32, "little")


def fe_from_bytes(b: bytes, mod: int) -> int:
    v = int.from_bytes(b, "little")
    if v >= mod:
        raise ValueError("non-canonical residue")
    return from_mont(v, mod)


def fr_to_bytes(x: int) -> bytes:
    return fe_to_bytes(x, R)


def fr_from_bytes(b: bytes) -> int:
    return fe_from_bytes(b, R)


def fr_vec_to_bytes(xs) -> bytes:
    return b"".join(fr_to_bytes(x) for x in xs)


def fr_vec_from_bytes(b: bytes):
    assert len(b) % 32 == 0
    return [fr_from_bytes(b[i:i + 32]) for i in range(0, len(b), 32)]


def int_to_fr(x: int) -> int:
    """Signed machine integer -> Fr (negatives map to r - |x|); src/fr-tensor.cu:30-39."""
    return x % R


# ----------------------------------------------------------------------------- curve (affine API)
INF = None  # affine infinity


def is_on_curve(pt) -> bool:
    if pt is INF:
        return True
    x, y = pt
    return (y * y - x * x * x - CURVE_B) % P == 0


def neg(pt):
    if pt is INF:
        return INF
    return (pt[0], (-pt[1]) % P)


def _jac_dbl(X, Y, Z):
    if Z == 0 or Y == 0:
        return (1, 1, 0)
    A = X * X % P
    B = Y * Y % P
    C = B * B % P
    D = 2 * ((X + B) * (X + B) - A - C) % P
    E = 3 * A % P
    F = E * E % P
    X3 = (F - 2 * D) % P
    Y3 = (E * (D - X3) - 8 * C) % P
    Z3 = 2 * Y * Z % P
    return (X3, Y3, Z3)


def _jac_add(p, q):
    X1, Y1, Z1 = p
    X2, Y2, Z2 = q
    if Z1 == 0:
        return q
    if Z2 == 0:
        return p
    Z1Z1 = Z1 * Z1 % P
    Z2Z2 = Z2 * Z2 % P
    U1 = X1 * Z2Z2 % P
    U2 = X2 * Z1Z1 % P
    S1 = Y1 * Z2 * Z2Z2 % P
    S2 = Y2 * Z1 * Z1Z1 % P
    if U1 == U2:
        if S1 == S2:
            return _jac_dbl(X1, Y1, Z1)
        return (1, 1, 0)
    H = (U2 - U1) % P
    Rr = (S2 - S1) % P
    HH = H * H % P
    HHH = H * HH % P
    V = U1 * HH % P
    X3 = (Rr * Rr - HHH - 2 * V) % P
    Y3 = (Rr * (V - X3) - S1 * HHH) % P
    Z3 = Z1 * Z2 * H % P
    return (X3, Y3, Z3)


def _to_jac(pt):
    return (1, 1, 0) if pt is INF else (pt[0], pt[1], 1)


def _from_jac(j):
    X, Y, Z = j
    if Z == 0:
        return INF
    zi = pow(Z, -1, P)
    zi2 = zi * zi % P
    return (X * zi2 % P, Y * zi2 * zi % P)


def add(p, q):
    return _from_jac(_jac_add(_to_jac(p), _to_jac(q)))


def scalar_mul(k: int, pt):
    """k*pt for any integer k (reduced mod the group order r)."""
    k %= R
    acc = (1, 1, 0)
    base = _to_jac(pt)
    while k:
        if k & 1:
            acc = _jac_add(acc, base)
        base = _jac_dbl(*base)
        k >>= 1
    return _from_jac(acc)


def msm(scalars, points):
    """sum_i scalars[i] * points[i] with signed Python-int scalars (bucket method, 8-bit windows).

    Any algorithm that yields the same group element conforms (src/Hyrax.cu:312-359 computes it
    with a fixed-base byte-window table); the result is returned normalised to affine.
    """
    assert len(scalars) == len(points)
    pairs = []
    maxbits = 1
    for s, pt in zip(scalars, points):
        if pt is INF:
            continue
        if abs(s) >= R:
            s %= R
        if s < 0:
            s, pt = -s, neg(pt)
        if s:
            pairs.append((s, _to_jac(pt)))
            maxbits = max(maxbits, s.bit_length())
    nwin = (maxbits + 7) // 8
    total = (1, 1, 0)
    for w in range(nwin - 1, -1, -1):
        for _ in range(8):
            total = _jac_dbl(*total)
        buckets = [None] * 256
        for s, jp in pairs:
            d = (s >> (8 * w)) & 255
            if d:
                buckets[d] = jp if buckets[d] is None else _jac_add(buckets[d], jp)
        run = (1, 1, 0)
        acc = (1, 1, 0)
        for d in range(255, 0, -1):
            if buckets[d] is not None:
                run = _jac_add(run, buckets[d])
            acc = _jac_add(acc, run)
        total = _jac_add(total, acc)
    return _from_jac(total)


# ----------------------------------------------------------------------------- point byte formats
def affine_to_bytes(pt) -> bytes:
    if pt is INF:
        return bytes(64)
    return fe_to_bytes(pt[0], P) + fe_to_bytes(pt[1], P)


def affine_from_bytes(b: bytes):
    assert len(b) == 64
    if b == bytes(64):
        return INF
    return (fe_from_bytes(b[:32], P), fe_from_bytes(b[32:], P))


def jacobian_to_bytes(pt) -> bytes:
    """Canonical 96-byte record: (x, y, 1) in Montgomery form, all-zero Z for infinity."""
    if pt is INF:
        return fe_to_bytes(1, P) + fe_to_bytes(1, P) + bytes(32)
    return fe_to_bytes(pt[0], P) + fe_to_bytes(pt[1], P) + fe_to_bytes(1, P)


def jacobian_from_bytes(b: bytes):
    """Any Jacobian representative -> normalised affine point (None for infinity)."""
    assert len(b) == 96
    X = fe_from_bytes(b[:32], P)
    Y = fe_from_bytes(b[32:64], P)
    Z = fe_from_bytes(b[64:], P)
    return _from_jac((X, Y, Z))


def jacobian_vec_from_bytes(b: bytes):
    assert len(b) % 96 == 0
    return [jacobian_from_bytes(b[i:i + 96]) for i in range(0, len(b), 96)]


# ----------------------------------------------------------------------------- seeded randomness
MASK64 = (1 << 64) - 1


class SplitMix64:
    """SplitMix64 stream; the same few lines exist in the C oracle and in the product's RNG seam."""

    def __init__(self, seed: int, tag: int = 0):
        self.state = (seed * 0x9E3779B97F4A7C15 + tag * 0xD1B54A32D192ED03 + 0x632BE59BD9B4E019) & MASK64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def next_fr(self) -> int:
        """512 random bits (eight little-endian 64-bit words) reduced mod r."""
        v = 0
        for i in range(8):
            v |= self.next_u64() << (64 * i)
        return v % R

    def fr_vec(self, n: int):
        return [self.next_fr() for _ in range(n)]


def make_generators(n: int, seed: int, tag: int = 1):
    """G_i = [rho_i] * (1, 2) with rho_i drawn from the seeded stream."""
    rng = SplitMix64(seed, tag)
    return [scalar_mul(rng.next_fr(), G1_GEN) for _ in range(n)]
