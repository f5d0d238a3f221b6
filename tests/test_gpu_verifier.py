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


@pytest.mark.parametrize("mapping", [False, True])
def test_lookup_proof_verifies_with_openings_of_A_and_m(gctx, mapping):
    """A lookup proof checked end to end by the verifier: round polynomials and closing identity
    (``verify_lookup``), the table evaluations recomputed from the public table, and the claimed A~(v),
    m~(v_low) tied to the commitments of A and m by Hyrax openings (``verify_open``)."""
    import grape_b200 as g
    from grape_b200 import host, verifier, workloads as wl
    rng = np.random.default_rng(17 + mapping)
    D, N, low, msm = 1 << 12, 1 << 8, -(1 << 7), 16
    wd = msm * 16
    gens_j = wl.make_generators(gctx, 256, seed=21)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    gctx.seed(600 + mapping)
    mapped = rng.integers(-1000, 1000, size=N).astype(np.int32) if mapping else None
    lk = host.Lookup(gctx, low, N, mapped)
    q = rng.integers(low, low + N, size=D).astype(np.int32)
    v = host.decode_field(gctx.random_fr(12))
    dS, dA = gctx.alloc(D * 32), gctx.alloc(D * 32)
    gctx.fr_from_i32(gctx.upload(q), D, dS)
    com_A, com_m = gctx.alloc(D // wd * 96), gctx.alloc(96)     # m: one row of 2^(8/2) * 16 = 256 multiplicities
    if mapping:
        d_out, work = gctx.alloc(D * 32), gctx.alloc(D * 32)
        gctx.fr_from_i32(gctx.upload(mapped[q - low]), D, d_out)
        claim, tr = lk.prove_pairs(dS, d_out, D, work, dA, v, table=table, msm_size=msm, d_com_A=com_A, d_com_m=com_m)
        S_vals = [(int(a) + lk.r * int(b)) % R for a, b in zip(q, mapped[q - low])]
    else:
        claim, tr = lk.prove(dS, D, dA, v, table=table, msm_size=msm, d_com_A=com_A, d_com_m=com_m)
        S_vals = [int(x) % R for x in q]
    finals, u = lk.last_proof()
    assert finals["S"] == claim == _mle(S_vals, v)
    te = verifier.lookup_table_evals(low, N, lk.beta, v[:8], mapped, lk.r if mapping else 0)
    assert verifier.verify_lookup(lk.alpha, lk.beta, N, D, tr, u, v, finals, te)
    bad = dict(finals, m=(finals["m"] + 1) % R)
    assert not verifier.verify_lookup(lk.alpha, lk.beta, N, D, tr, u, v, bad, te)
    tr2 = [list(p) for p in tr]
    tr2[5][2] = (tr2[5][2] + 1) % R
    assert not verifier.verify_lookup(lk.alpha, lk.beta, N, D, tr2, u, v, finals, te)
    # A~(v) against the commitment of A: the prover rebuilds A = 1 / (S + beta) and opens it at v
    A_vals = [pow((s + lk.beta) % R, -1, R) for s in S_vals]
    c = int(rng.integers(1, 2**62))
    proof = host.hyrax_open(gctx, table, gctx.fr_upload(A_vals), D, msm, 1, v, c, gens_j[0])
    assert proof["result"] == finals["A"]
    com_rows = gctx.download(com_A, D // wd * 96).reshape(-1, 24)
    assert verifier.verify_open(gctx, table, com_rows, proof, v, c, D, msm, 1, gens_j[0])
    # m~(v_low) against the commitment of m (one row of 256 multiplicities)
    m_vals = lk.table("m")
    proof_m = host.hyrax_open(gctx, table, gctx.fr_upload(m_vals), N, 16, 1, v[:8], c, gens_j[0])
    assert proof_m["result"] == finals["m"]
    com_m_rows = gctx.download(com_m, 96).reshape(-1, 24)
    assert verifier.verify_open(gctx, table, com_m_rows, proof_m, v[:8], c, N, 16, 1, gens_j[0])
    lk.close()
    table.close()


def test_unseeded_contexts_draw_different_blinders_and_still_verify():
    """A context that was never seeded takes its randomness from the operating system: two of them open
    the same tensor at the same point with different z vectors, and both openings verify."""
    import grape_b200 as g
    from grape_b200 import host, verifier, workloads as wl
    rng = random.Random(2)
    N, layer_num, rows = 2, 1, 2
    wd = N * 16
    size = layer_num * rows * wd
    t = np.array([rng.randrange(-2**31, 2**31) for _ in range(size)], dtype=np.int32)
    e = [rng.randrange(R) for _ in range(pr.log2ceil(size))]
    c = rng.randrange(R)
    zs = []
    for _ in range(2):
        ctx = g.Context(0)
        seeded = g.Context(0)
        gens_j = wl.make_generators(seeded, wd, seed=5)     # generators: a seeded helper context
        seeded.close()
        table = g.GeneratorTable(ctx, gens_j, 8, 1)
        d_int = ctx.upload(t)
        com = ctx.alloc(rows * 96)
        g.commit_i32(ctx, table, d_int, size, wd, com)
        commitments = ctx.download(com, rows * 96).reshape(-1, 24)
        d_t = ctx.alloc(size * 32)
        ctx.fr_from_i32(d_int, size, d_t)
        proof = host.hyrax_open(ctx, table, d_t, size, N, layer_num, e, c, gens_j[0])
        assert verifier.verify_open(ctx, table, commitments, proof, e, c, size, N, layer_num, gens_j[0])
        zs.append(proof.z_raw.tobytes())
        draws = ctx.random_fr(4)
        assert len({draws[k].tobytes() for k in range(4)}) == 4
        table.close()
        ctx.close()
    assert zs[0] != zs[1]
