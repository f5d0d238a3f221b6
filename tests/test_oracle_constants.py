"""The oracle's moduli and Montgomery constants equal the reference's literals
(include/field/alt_bn128.cuh:11-45, written there as 64-bit halves)."""
from oracle import bn254


def _join(words):
    return sum(w << (64 * i) for i, w in enumerate(words))


def test_moduli_and_montgomery_constants():
    P = _join([0x3c208c16d87cfd47, 0x97816a916871ca8d, 0xb85045b68181585d, 0x30644e72e131a029])
    RR = _join([0xf32cfc5b538afa89, 0xb5e71911d44501fb, 0x47ab1eff0a417ff6, 0x06d89f71cab8351f])
    ONE = _join([0xd35d438dc58f0d9d, 0x0a78eb28f5c70b3d, 0x666ea36f7879462c, 0x0e0a77c19a07df2f])
    r = _join([0x43e1f593f0000001, 0x2833e84879b97091, 0xb85045b68181585d, 0x30644e72e131a029])
    rRR = _join([0x1bb8e645ae216da7, 0x53fe3ab1e35c59e3, 0x8c49833d53bb8085, 0x0216d0b17f4e44a5])
    rone = _join([0xac96341c4ffffffb, 0x36fc76959f60cd29, 0x666ea36f7879462e, 0x0e0a77c19a07df2f])
    assert bn254.P == P and bn254.R == r
    assert pow(2, 512, P) == RR and pow(2, 256, P) == ONE
    assert pow(2, 512, r) == rRR and pow(2, 256, r) == rone
    assert (-pow(P, -1, 2**32)) % 2**32 == 0xe4866389
    assert (-pow(r, -1, 2**32)) % 2**32 == 0xefffffff
    assert bn254.is_on_curve(bn254.G1_GEN)
    assert bn254.scalar_mul(bn254.R, bn254.G1_GEN) is None  # r is the group order


def test_byte_formats_roundtrip():
    g5 = bn254.scalar_mul(5, bn254.G1_GEN)
    assert bn254.affine_from_bytes(bn254.affine_to_bytes(g5)) == g5
    assert bn254.affine_from_bytes(bytes(64)) is None
    assert bn254.jacobian_from_bytes(bn254.jacobian_to_bytes(g5)) == g5
    assert bn254.jacobian_from_bytes(bn254.jacobian_to_bytes(None)) is None
    assert bn254.fr_from_bytes(bn254.fr_to_bytes(-7)) == bn254.R - 7
