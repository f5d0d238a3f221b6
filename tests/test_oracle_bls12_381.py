"""The BLS12-381 oracle's constants equal the reference's literals (include/field/bls12-381.cuh:7-46,
written there as 64-bit halves) and the curve's public parameters hold."""
from oracle import bls12_381 as bls


def _join(words):
    return sum(w << (64 * i) for i, w in enumerate(words))


def test_moduli_and_montgomery_constants():
    P = _join([0xb9feffffffffaaab, 0x1eabfffeb153ffff, 0x6730d2a0f6b0f624, 0x64774b84f38512bf,
               0x4b1ba7b6434bacd7, 0x1a0111ea397fe69a])
    RR = _join([0xf4df1f341c341746, 0x0a76e6a609d104f1, 0x8de5476c4c95b6d5, 0x67eb88a9939d83c0,
                0x9a793e85b519952d, 0x11988fe592cae3aa])
    ONE = _join([0x760900000002fffd, 0xebf4000bc40c0002, 0x5f48985753c758ba, 0x77ce585370525745,
                 0x5c071a97a256ec6d, 0x15f65ec3fa80e493])
    r = _join([0xffffffff00000001, 0x53bda402fffe5bfe, 0x3339d80809a1d805, 0x73eda753299d7d48])
    rRR = _join([0xc999e990f3f29c6d, 0x2b6cedcb87925c23, 0x05d314967254398f, 0x0748d9d99f59ff11])
    rone = _join([0x00000001fffffffe, 0x5884b7fa00034802, 0x998c4fefecbc4ff5, 0x1824b159acc5056f])
    assert bls.P == P and bls.R == r
    assert pow(2, 768, P) == RR and pow(2, 384, P) == ONE
    assert pow(2, 512, r) == rRR and pow(2, 256, r) == rone
    assert (-pow(P, -1, 2**32)) % 2**32 == 0xfffcfffd
    assert (-pow(r, -1, 2**32)) % 2**32 == 0xffffffff


def test_generator_and_group_order():
    assert bls.is_on_curve(bls.G1_GEN)
    assert bls.scalar_mul(bls.R, bls.G1_GEN) is None
    assert bls.scalar_mul(bls.R - 1, bls.G1_GEN) == bls.neg(bls.G1_GEN)


def test_msm_and_byte_formats():
    g = [bls.scalar_mul(k, bls.G1_GEN) for k in (3, 5, 7, 11)]
    assert bls.msm([2, -3, 70000, 0], g) == bls.scalar_mul(2 * 3 - 3 * 5 + 70000 * 7, bls.G1_GEN)
    assert bls.msm([1, 1, -1, 0], [g[0], g[0], g[0], g[1]]) == g[0]
    assert bls.msm([5, -3], g[:2]) is None  # 5*3 - 3*5
    assert bls.jacobian_from_bytes(bls.jacobian_to_bytes(g[2])) == g[2]
    assert bls.jacobian_from_bytes(bls.jacobian_to_bytes(None)) is None
    assert bls.fr_from_bytes(bls.fr_to_bytes(-7)) == bls.R - 7
    assert len(bls.jacobian_to_bytes(g[0])) == 144
    rows = bls.commit_rows([1, 2, 3, 4, -1, 0, 0, 9], 4, g)
    assert rows[0] == bls.scalar_mul(1 * 3 + 2 * 5 + 3 * 7 + 4 * 11, bls.G1_GEN)
    assert rows[1] == bls.scalar_mul(-3 + 9 * 11, bls.G1_GEN)
