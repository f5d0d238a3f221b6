"""The verifier accepts what the provers produce and rejects tampered proofs."""
import random

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def test_lincomb_matches_oracle(gctx):
    import grape_b200 as g
    from grape_b200 import verifier
    rng = random.Random(1)
    pts = [bn254.scalar_mul(rng.randrange(R), bn254.G1_GEN) for _ in range(37)] + [None, bn254.G1_GEN]
    sc = [rng.randrange(R) for _ in range(37)] + [5, 0]
    got = verifier.lincomb(gctx, g.encode_jacobian(pts), sc)
    assert got == bn254.jacobian_to_bytes(bn254.msm(sc, pts))
    assert verifier.lincomb(gctx, g.encode_jacobian([bn254.G1_GEN, bn254.neg(bn254.G1_GEN)]), [7, 7]) == \
        bn254.jacobian_to_bytes(None)


@pytest.mark.parametrize("layer_num,N,rows", [(2, 2, 2), (1, 4, 3), (4, 1, 1)])
def test_open_verifies_and_tampering_fails(gctx, layer_num, N, rows):
    import grape_b200 as g
    from grape_b200 import host, verifier, workloads as wl
    rng = random.Random(N)
    wd = N * 16
    gens_j = wl.make_generators(gctx, wd, seed=5)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    size = layer_num * rows * wd
    t = np.array([rng.randrange(-2**31, 2**31) for _ in range(size)], dtype=np.int32)
    d_int = gctx.upload(t)
    com = gctx.alloc((size // wd) * 96)
    g.commit_i32(gctx, table, d_int, size, wd, com)
    commitments = gctx.download(com, (size // wd) * 96).reshape(-1, 24)
    d_t = gctx.alloc(size * 32)
    gctx.fr_from_i32(d_int, size, d_t)
    e = [rng.randrange(R) for _ in range(pr.log2ceil(size))]
    c = rng.randrange(R)
    proof = host.hyrax_open(gctx, table, d_t, size, N, layer_num, e, c, gens_j[0])
    assert proof["result"] == _mle([int(x) % R for x in t], e)
    assert verifier.verify_open(gctx, table, commitments, proof, e, c, size, N, layer_num, gens_j[0])
    bad = host.OpenProof(proof.result_raw.copy(), proof.z_raw.copy(), proof.com_raw.copy())
    bad.z_raw[3, 0] ^= 1
    assert not verifier.verify_open(gctx, table, commitments, bad, e, c, size, N, layer_num, gens_j[0])
    bad = host.OpenProof(host.encode_field([(proof["result"] + 1) % R]), proof.z_raw, proof.com_raw)
    assert not verifier.verify_open(gctx, table, commitments, bad, e, c, size, N, layer_num, gens_j[0])
    other = commitments.copy()
    other[0] = commitments[-1] if len(commitments) > 1 else g.encode_jacobian([bn254.G1_GEN])[0]
    if len(commitments) > 1:
        assert not verifier.verify_open(gctx, table, other, proof, e, c, size, N, layer_num, gens_j[0])
    table.close()


def test_sumcheck_transcripts_verify(gctx):
    from grape_b200 import host, verifier
    rng = random.Random(9)
    L, N, M, K = 2, 4, 8, 11
    A = [rng.randrange(-2**15, 2**15) % R for _ in range(L * N * K)]
    B = [rng.randrange(-2**15, 2**15) % R for _ in range(L * M * K)]
    u = [rng.randrange(R) for _ in range(3 + 2 + 1)]
    v = [rng.randrange(R) for _ in range(4 + 1)]
    Y = [sum(A[(l * N + n) * K + k] * B[(l * M + m) * K + k] for k in range(K)) % R
         for l in range(L) for n in range(N) for m in range(M)]
    claim = _mle(Y, u)
    a, b, final, tr = host.prove_matmul(gctx, gctx.fr_upload(A), gctx.fr_upload(B), L, N, M, K, u, v, claim)
    assert verifier.verify_matmul(claim, tr, u, v, L, N, M, K, a, b)
    assert not verifier.verify_matmul(claim, tr, u, v, L, N, M, K, a, (b + 1) % R)
    tr2 = [list(p) for p in tr]
    tr2[1][0] = (tr2[1][0] + 1) % R
    assert not verifier.verify_matmul(claim, tr2, u, v, L, N, M, K, a, b)
    # Hadamard product (power-of-two inner dimension) and claim batching
    n = 64
    X = [rng.randrange(R) for _ in range(n)]
    Z = [rng.randrange(R) for _ in range(n)]
    uu = [rng.randrange(R) for _ in range(6)]
    vv = [rng.randrange(R) for _ in range(6)]
    cl = _mle([x * z % R for x, z in zip(X, Z)], uu)
    a, b, final, tr = host.prove_elemul(gctx, gctx.fr_upload(X), gctx.fr_upload(Z), 2, 4, 8, uu, vv, cl)
    assert verifier.verify_elemul(cl, tr, uu, vv, a, b) and not verifier.verify_elemul(cl, tr, uu, vv, b, (a + 1) % R)
    us = [[rng.randrange(R) for _ in range(6)] for _ in range(3)]
    claims = [_mle(X, uj) for uj in us]
    res, tr = host.combine_claims(gctx, gctx.fr_upload(X), n, claims, us, vv)
    assert verifier.verify_combine(claims, tr, us, vv, res)
    assert not verifier.verify_combine(claims, tr, us, vv, (res + 1) % R)
