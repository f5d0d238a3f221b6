"""The transcript verifier's host arithmetic against the oracle's provers (no GPU): accepted transcripts,
and the rejections a verifier owes its caller (wrong lengths, extra coefficients, tampered values)."""
import random

import pytest

from oracle import bn254
from oracle import protocols as pr

R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


@pytest.mark.parametrize("low,N,D,mapped", [(-8, 16, 64, False), (-4, 8, 8, False), (-8, 16, 128, True), (-2, 4, 4096, False)])
def test_lookup_transcript_verifies_and_tampering_fails(low, N, D, mapped):
    from grape_b200 import verifier as V
    rng = random.Random(N * 1000 + D)
    alpha = rng.randrange(R)
    v = [rng.randrange(R) for _ in range(pr.log2ceil(D))]
    u = [rng.randrange(R) for _ in v]
    if mapped:
        mp = [rng.randrange(-100, 100) for _ in range(N)]
        lk = pr.LookupRangeMapping(low, N, mp, alpha, rng.randrange(R))
        s_in = [rng.randrange(low, low + N) for _ in range(D)]
        out = lk.prove_pairs([s % R for s in s_in], [mp[s - low] % R for s in s_in], v, u)
    else:
        mp = None
        lk = pr.LookupRange(low, N, alpha)
        out = lk.prove([rng.randrange(low, low + N) % R for _ in range(D)], v, u)
    lN = pr.log2ceil(N)
    fin = {"A": V.mle_eval(out["A"], v), "S": V.mle_eval(out["S_padded"], v), "B": V.mle_eval(lk.B, v[:lN]),
           "T": V.mle_eval(lk.T, v[:lN]), "m": V.mle_eval(out["m"], v[:lN])}
    assert fin["S"] == out["claim"]
    te = V.lookup_table_evals(low, N, lk.beta, v[:lN], mp, lk.r if mapped else 0)
    assert te == (fin["T"], fin["B"])        # the verifier's own evaluation of the public table
    args = (alpha, lk.beta, N, D)
    assert V.verify_lookup(*args, out["transcript"], u, v, fin, te)
    for key in ("A", "S", "m"):
        bad = dict(fin)
        bad[key] = (bad[key] + 1) % R
        assert not V.verify_lookup(*args, out["transcript"], u, v, bad, te)
    bad = dict(fin)
    bad["B"] = (bad["B"] + 1) % R            # caught by the table evaluation, not by the identity alone
    assert not V.verify_lookup(*args, out["transcript"], u, v, bad, te)
    tr = [list(p) for p in out["transcript"]]
    tr[len(tr) // 2][1] = (tr[len(tr) // 2][1] + 1) % R
    assert not V.verify_lookup(*args, tr, u, v, fin, te)
    assert not V.verify_lookup(*args, out["transcript"][:-1], u, v, fin, te)             # a round missing
    assert not V.verify_lookup(*args, out["transcript"], u[:-1], v, fin, te)
    long = [list(p) for p in out["transcript"]]
    long[0] = long[0] + [0] * (5 - len(long[0]))                                          # a fifth coefficient
    assert not V.verify_lookup(*args, long, u, v, fin, te)
    assert not V.verify_lookup((alpha + 1) % R, lk.beta, N, D, out["transcript"], u, v, fin, te)


def test_sumcheck_verifiers_reject_malformed_transcripts():
    from grape_b200 import verifier as V
    rng = random.Random(3)
    L, N, M, K = 2, 2, 4, 6
    A = [rng.randrange(-2**15, 2**15) % R for _ in range(L * N * K)]
    B = [rng.randrange(-2**15, 2**15) % R for _ in range(L * M * K)]
    u = [rng.randrange(R) for _ in range(2 + 1 + 1)]
    v = [rng.randrange(R) for _ in range(3 + 1)]
    Y = [sum(A[(l * N + n) * K + k] * B[(l * M + m) * K + k] for k in range(K)) % R
         for l in range(L) for n in range(N) for m in range(M)]
    claim = _mle(Y, u)
    a, b, final, tr = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
    assert V.verify_matmul(claim, tr, u, v, L, N, M, K, a, b)
    assert not V.verify_matmul(claim, tr[:-1], u, v, L, N, M, K, a, b)                    # truncated
    assert not V.verify_matmul((claim + 1) % R, tr, u, v, L, N, M, K, a, b)               # wrong claim
    assert not V.verify_matmul(claim, tr, u[:-1], v, L, N, M, K, a, b)                    # short challenge vector
    extra = [list(p) for p in tr]
    extra[-1] = extra[-1] + [0] * (3 - len(extra[-1])) + [1]                              # a cubic term in a quadratic round
    assert not V.verify_matmul(claim, extra, u, v, L, N, M, K, a, b)
    # Hadamard product: the number of rounds is tied to the tensor size
    n = 32
    X = [rng.randrange(R) for _ in range(n)]
    Z = [rng.randrange(R) for _ in range(n)]
    uu = [rng.randrange(R) for _ in range(5)]
    vv = [rng.randrange(R) for _ in range(5)]
    cl = _mle([x * z % R for x, z in zip(X, Z)], uu)
    a, b, final, tr = pr.prove_elemul(X, Z, 2, 2, 8, uu, vv, cl)
    assert V.verify_elemul(cl, tr, uu, vv, a, b, size=n)
    assert not V.verify_elemul(cl, tr, uu, vv, a, b, size=2 * n)
    assert not V.verify_elemul(cl, [], uu, vv, a, b)                                      # an empty transcript proves nothing
    assert not V.verify_elemul(cl, tr[:3], uu[:3], vv[:3], a, b, size=n)
    assert not V.verify_elemul(cl, tr, uu, vv, a, (b + 1) % R, size=n)
    # claim batching: every point must have the length of v
    us = [[rng.randrange(R) for _ in range(5)] for _ in range(2)]
    claims = [_mle(X, uj) for uj in us]
    res, tr = pr.combine_claims(X, claims, us, vv, n)
    assert V.verify_combine(claims, tr, us, vv, res)
    assert not V.verify_combine(claims, tr, [us[0], us[1][:-1]], vv, res)
    assert not V.verify_combine(claims[:1], tr, us, vv, res)
    assert not V.verify_combine(claims, tr, us, vv, (res + 1) % R)
