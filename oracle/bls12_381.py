"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the BLS12-381 instantiation of the commitment path.

The reference ships field constants for BLS12-381 (include/field/bls12-381.cuh:7-46: a 381-bit base
field on twelve 32-bit limbs with Montgomery radix 2^384, a 255-bit scalar field on eight limbs with
radix 2^256) but compiles none of its code against them, so there is no reference output to compare
with on this curve.  This module restates the published curve (y^2 = x^3 + 4 over Fp, the standard
G1 generator, group order r) on Python integers with the same record layouts the BN254 path uses,
scaled to 48-byte coordinates: affine 96 B (X|Y, (0,0) = infinity), Jacobian 144 B (X|Y|Z, Z = 0 =
infinity), all coordinates Montgomery residues as little-endian 32-bit limbs.

Parity status for this curve: pinned to the reference's constants and to the curve's public
parameters (generator on the curve, r * G = infinity); no reference run exists to pin outputs to.
"""
from __future__ import annotations

P = 0x1A0111EA397FE69A4B1BA7B6434BACD764774B84F38512BF6730D2A0F6B0F6241EABFFFEB153FFFFB9FEFFFFFFFFAAAB
R = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001
FP_BYTES = 48
FR_BYTES = 32
MONT_P = 1 << 384
MONT_R = 1 << 256
CURVE_B = 4
G1_GEN = (
    0x17F1D3A73197D7942695638C4FA9AC0FC3688C4F9774B905A14E3A3F171BAC586C55E83FF97A1AEFFB3AF00ADB22C6BB,
    0x08B3F481E3AAA0F1A09E30ED741D8AE4FCF5E095D5D00AF600DB18CB2C04B3EDD03CC744A2888AE40CAA232946C5E7E1,
)
INF = None

_RINV_P = pow(MONT_P, -1, P)
_RINV_R = pow(MONT_R, -1, R)


def fp_to_bytes(x: int) -> bytes:
    return ((x % P) * MONT_P % P).to_bytes(FP_BYTES, "little")


def fp_from_bytes(b: bytes) -> int:
    return int.from_bytes(b, "little") * _RINV_P % P


def fr_to_bytes(x: int) -> bytes:
    return ((x % R) * MONT_R % R).to_bytes(FR_BYTES, "little")


def fr_from_bytes(b: bytes) -> int:
    return int.from_bytes(b, "little") * _RINV_R % R


def is_on_curve(pt) -> bool:
    if pt is None:
        return True
    x, y = pt
    return (y * y - x * x * x - CURVE_B) % P == 0


def neg(pt):
    return None if pt is None else (pt[0], (-pt[1]) % P)


def _dbl(X, Y, Z):
    if Z == 0 or Y == 0:
        return (1, 1, 0)
    A = X * X % P
    B = Y * Y % P
    C = B * B % P
    D = 2 * ((X + B) * (X + B) - A - C) % P
    E = 3 * A % P
    X3 = (E * E - 2 * D) % P
    Y3 = (E * (D - X3) - 8 * C) % P
    Z3 = 2 * Y * Z % P
    return (X3, Y3, Z3)


def _add(p, q):
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
        return _dbl(X1, Y1, Z1) if S1 == S2 else (1, 1, 0)
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
    return (1, 1, 0) if pt is None else (pt[0], pt[1], 1)


def _from_jac(j):
    X, Y, Z = j
    if Z == 0:
        return None
    zi = pow(Z, -1, P)
    return (X * zi * zi % P, Y * zi * zi * zi % P)


def add(p, q):
    return _from_jac(_add(_to_jac(p), _to_jac(q)))


def scalar_mul(k: int, pt):
    """[k] pt for any integer k (negative k negates the point)."""
    if pt is None or k == 0:
        return None
    if k < 0:
        return scalar_mul(-k, neg(pt))
    acc = (1, 1, 0)
    base = _to_jac(pt)
    for bit in bin(k)[2:]:
        acc = _dbl(*acc)
        if bit == "1":
            acc = _add(acc, base)
    return _from_jac(acc)


def msm(scalars, points):
    """sum_i [s_i] P_i with signed integer scalars (bucket method over 8-bit windows)."""
    acc = (1, 1, 0)
    pairs = [(s, p) if s >= 0 else (-s, neg(p)) for s, p in zip(scalars, points) if s != 0 and p is not None]
    if not pairs:
        return None
    top = max(s.bit_length() for s, _ in pairs)
    c = 8
    for w in reversed(range((top + c - 1) // c)):
        for _ in range(c):
            acc = _dbl(*acc)
        buckets = [(1, 1, 0)] * (1 << c)
        for s, p in pairs:
            d = (s >> (c * w)) & ((1 << c) - 1)
            if d:
                buckets[d] = _add(buckets[d], _to_jac(p))
        run = (1, 1, 0)
        tot = (1, 1, 0)
        for d in range((1 << c) - 1, 0, -1):
            run = _add(run, buckets[d])
            tot = _add(tot, run)
        acc = _add(acc, tot)
    return _from_jac(acc)


def commit_rows(scalars, wd, gens):
    """Row commitments of a row-major tensor of signed integers (the Hyrax commit on this curve)."""
    return [msm(scalars[r:r + wd], gens[:wd]) for r in range(0, len(scalars), wd)]


def jacobian_to_bytes(pt) -> bytes:
    if pt is None:
        return fp_to_bytes(1) + fp_to_bytes(1) + bytes(FP_BYTES)
    return fp_to_bytes(pt[0]) + fp_to_bytes(pt[1]) + fp_to_bytes(1)


def jacobian_from_bytes(b: bytes):
    x, y, z = (fp_from_bytes(b[i * FP_BYTES:(i + 1) * FP_BYTES]) for i in range(3))
    return _from_jac((x, y, z))


def jacobian_vec_from_bytes(b: bytes):
    n = 3 * FP_BYTES
    return [jacobian_from_bytes(b[i:i + n]) for i in range(0, len(b), n)]


def affine_from_bytes(b: bytes):
    x, y = fp_from_bytes(b[:FP_BYTES]), fp_from_bytes(b[FP_BYTES:2 * FP_BYTES])
    return None if x == 0 and y == 0 else (x, y)
