"""Self-consistency of the protocol restatements (oracle/protocols.py): every round check of the
reference closes, final identities hold, and the returned claims equal independently computed
multilinear evaluations -- including non-power-of-two inner dimensions."""
import random

import pytest

from oracle import bn254 as b
from oracle import protocols as pr

R = b.R


def mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def pad_rows(X, rows, n):
    npad = 1 << pr.log2ceil(n)
    return [x for i in range(rows) for x in X[i * n:(i + 1) * n] + [0] * (npad - n)]


def test_fold_equals_eq_weight_sum():
    rng = random.Random(0)
    t = [rng.randrange(R) for _ in range(2 * 11 * 3)]
    x = [rng.randrange(R) for _ in range(4)]
    w = pr.eq_weights(x, 4, 11)
    want = [sum(w[j] * t[(o * 11 + j) * 3 + g] for j in range(11)) % R for o in range(2) for g in range(3)]
    assert pr.partial_eval(t, len(t), x, 11, 0, 3) == want


@pytest.mark.parametrize("L,N,M,K", [(1, 4, 8, 6), (2, 4, 2, 6), (4, 2, 4, 11), (1, 2, 2, 8)])
def test_matmul_sumcheck(L, N, M, K):
    rng = random.Random(L + N + M + K)
    draw = b.SplitMix64(7)
    A = [rng.randrange(-50, 50) % R for _ in range(L * N * K)]
    B = [rng.randrange(-50, 50) % R for _ in range(L * M * K)]
    Y = [sum(A[(l * N + n) * K + k] * B[(l * M + m) * K + k] for k in range(K)) % R
         for l in range(L) for n in range(N) for m in range(M)]
    u = draw.fr_vec(pr.log2ceil(L * N * M))
    v = draw.fr_vec(pr.log2ceil(L * K))
    a, bb, final, tr = pr.prove_matmul(A, B, L, N, M, K, u, v, mle(Y, u))
    u2, v2 = pr.reassemble_vectors(u, v, pr.log2ceil(N), pr.log2ceil(K), pr.log2ceil(M))
    assert mle(pad_rows(A, L * N, K), u2) == a
    assert mle(pad_rows(B, L * M, K), v2) == bb
    assert len(tr) == pr.log2ceil(L) + pr.log2ceil(K)
    with pytest.raises(RuntimeError):
        pr.prove_matmul(A, B, L, N, M, K, u, v, (mle(Y, u) + 1) % R)


@pytest.mark.parametrize("L,M,N", [(2, 2, 6), (1, 4, 4), (2, 2, 11)])
def test_hadamard_sumcheck(L, M, N):
    rng = random.Random(L * M * N)
    A = [rng.randrange(R) for _ in range(L * M * N)]
    B = [rng.randrange(R) for _ in range(L * M * N)]
    nv = pr.log2ceil(L * M * N)
    u = [rng.randrange(R) for _ in range(nv)]
    v = [rng.randrange(R) for _ in range(nv)]
    claim = mle(pad_rows([x * y % R for x, y in zip(A, B)], L * M, N), u)
    a, bb, final, tr = pr.prove_elemul(A, B, L, M, N, u, v, claim)
    assert a == mle(pad_rows(A, L * M, N), v) and bb == mle(pad_rows(B, L * M, N), v)


def test_combine_claims():
    rng = random.Random(3)
    X = [rng.randrange(R) for _ in range(16)]
    us = [[rng.randrange(R) for _ in range(4)] for _ in range(3)]
    v = [rng.randrange(R) for _ in range(4)]
    ret, tr = pr.combine_claims(X, [mle(X, uj) for uj in us], us, v, 16)
    assert ret == mle(X, v) and len(tr) == 4


def test_lookup_range_and_mapping():
    rng = random.Random(4)
    draw = b.SplitMix64(9)
    lk = pr.LookupRange(-8, 16, draw.next_fr())
    S = [rng.randrange(-8, 8) % R for _ in range(64)]
    v, u = draw.fr_vec(6), draw.fr_vec(6)
    out = lk.prove(S, v, u)
    assert out["claim"] == mle(S, v)
    assert sum(out["m"]) == 64 and len(out["transcript"]) == 6
    # a query outside the table breaks the very first round check
    bad = list(S)
    bad[3] = 100
    lk2 = pr.LookupRange(-8, 16, draw.next_fr())
    with pytest.raises((RuntimeError, IndexError)):
        lk2.prove(bad, v, u)
    mp = [rng.randrange(-100, 100) for _ in range(16)]
    lm = pr.LookupRangeMapping(-8, 16, mp, draw.next_fr(), draw.next_fr())
    s_in = [rng.randrange(-8, 8) for _ in range(32)]
    s_out = [mp[s + 8] % R for s in s_in]
    v, u = draw.fr_vec(5), draw.fr_vec(5)
    out = lm.prove_pairs([s % R for s in s_in], s_out, v, u)
    assert out["claim"] == mle([(a % R + lm.r * o) % R for a, o in zip(s_in, s_out)], v)


def test_hyrax_open_verifies():
    rng = random.Random(5)
    draw = b.SplitMix64(11)
    gens = b.make_generators(32, 5)
    layer_num, N, size = 2, 2, 128
    t = [rng.randrange(-1000, 1000) for _ in range(size)]
    com = pr.commit_rows(t, 32, gens)
    e, c, d = draw.fr_vec(7), draw.next_fr(), draw.fr_vec(32)
    proof = pr.hyrax_open([x % R for x in t], e, c, size, N, layer_num, gens, gens[0], d)
    assert proof["result"] == mle([x % R for x in t], e)
    assert pr.hyrax_verify(com, proof, e, c, size, N, layer_num, gens, gens[0])
    proof["z"][0] = (proof["z"][0] + 1) % R
    assert not pr.hyrax_verify(com, proof, e, c, size, N, layer_num, gens, gens[0])


@pytest.mark.parametrize("L,N,M,K,P", [(1, 4, 4, 8, 2), (2, 3, 4, 8, 4), (1, 2, 2, 12, 4), (4, 2, 3, 8, 8), (1, 2, 2, 24, 8)])
def test_sharded_matmul_sumcheck_equals_the_unsharded_one(L, N, M, K, P):
    """The inner dimension dealt to P provers by residue class: local rounds + one exchange + the last
    log2(P) rounds give the reference prover's transcript and claims, bit for bit."""
    import random
    rnd = random.Random(L * 1000 + K * 10 + P)
    A = [rnd.randrange(-50, 50) % R for _ in range(L * N * K)]
    B = [rnd.randrange(-50, 50) % R for _ in range(L * M * K)]
    u = [rnd.randrange(R) for _ in range(pr.log2ceil(L * N * M) + 1)]
    v = [rnd.randrange(R) for _ in range(pr.log2ceil(L * K))]
    a_ = pr.partial_eval(list(A), len(A), u, N, pr.log2ceil(M), K)
    b_ = pr.partial_eval(list(B), len(B), u, M, 0, K)
    lL, u_end = pr.log2ceil(L), pr.log2ceil(L * N * M)
    w = pr.eq_weights(u[u_end - lL:u_end], lL, L)
    claim = sum(w[l] * a_[l * K + k] * b_[l * K + k] for l in range(L) for k in range(K)) % R
    want = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
    lp = pr.log2ceil(P)
    parts = []
    for r in range(P):
        As = [A[(l * N + n) * K + k] for l in range(L) for n in range(N) for k in range(r, K, P)]
        Bs = [B[(l * M + m) * K + k] for l in range(L) for m in range(M) for k in range(r, K, P)]
        parts.append(pr.prove_matmul_partial(As, Bs, L, N, M, K // P, u, v[lp:]))
    assert pr.prove_matmul_finish(parts, L, N, M, K, u, v, claim) == want
    # a wrong claim is rejected by the round check, as in the reference
    with pytest.raises(RuntimeError):
        pr.prove_matmul_finish(parts, L, N, M, K, u, v, (claim + 1) % R)
