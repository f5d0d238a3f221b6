"""Parity of the sumcheck provers with the oracle: returned claims and every round polynomial."""
import random

import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def _pad4(polys):
    return [list(p) + [0] * (4 - len(p)) for p in polys]


@pytest.mark.parametrize("L,N,M,K", [(1, 4, 8, 6), (2, 4, 2, 6), (4, 2, 4, 11), (1, 2, 2, 8), (1, 16, 8, 300), (2, 4, 8, 64), (1, 3, 8, 33),
                                     (1, 2, 2, 9000), (2, 2, 2, 16384)])  # the last two start above the fused-tail size
def test_prove_matmul(gctx, L, N, M, K):
    from grape_b200 import host
    rng = random.Random(L * 1000 + N * 100 + M * 10 + K)
    draw = bn254.SplitMix64(K, 5)
    A = [rng.randrange(-2**15, 2**15) % R for _ in range(L * N * K)]
    B = [rng.randrange(-2**15, 2**15) % R for _ in range(L * M * K)]
    u = draw.fr_vec(pr.log2ceil(M) + pr.log2ceil(N) + pr.log2ceil(L))
    v = draw.fr_vec(pr.log2ceil(K) + pr.log2ceil(L))
    Mp, Np = 1 << pr.log2ceil(M), 1 << pr.log2ceil(N)
    Y = [0] * (L * Np * Mp)
    for l in range(L):
        for n in range(N):
            for m in range(M):
                Y[(l * Np + n) * Mp + m] = sum(A[(l * N + n) * K + k] * B[(l * M + m) * K + k] for k in range(K)) % R
    claim = _mle(Y, u)
    want = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
    dA, dB = gctx.fr_upload(A), gctx.fr_upload(B)
    got = host.prove_matmul(gctx, dA, dB, L, N, M, K, u, v, claim)
    assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
    assert got[3] == _pad4(want[3])
    # the same proof straight from the int32 tensors
    import numpy as np
    to_i32 = lambda X: np.array([x if x < R // 2 else x - R for x in X], dtype=np.int32)
    got_i = host.prove_matmul_i32(gctx, gctx.upload(to_i32(A)), gctx.upload(to_i32(B)), L, N, M, K, u, v, claim)
    assert got_i == got


def test_prove_matmul_rejects_wrong_claim(gctx):
    import grape_b200 as g
    from grape_b200 import host
    rng = random.Random(5)
    L, N, M, K = 1, 2, 2, 4
    A = [rng.randrange(R) for _ in range(L * N * K)]
    B = [rng.randrange(R) for _ in range(L * M * K)]
    u = [rng.randrange(R) for _ in range(2)]
    v = [rng.randrange(R) for _ in range(2)]
    with pytest.raises(g.GrapeError) as e:
        host.prove_matmul(gctx, gctx.fr_upload(A), gctx.fr_upload(B), L, N, M, K, u, v, 12345)
    assert e.value.code == 3  # GRAPE_ERR_CHECK, the reference throws std::runtime_error here


@pytest.mark.parametrize("L,M,N", [(2, 2, 6), (1, 4, 4), (2, 2, 11), (1, 1, 8), (4, 8, 37)])
def test_prove_elemul(gctx, L, M, N):
    from grape_b200 import host
    rng = random.Random(L * 100 + M * 10 + N)
    A = [rng.randrange(R) for _ in range(L * M * N)]
    B = [rng.randrange(R) for _ in range(L * M * N)]
    Np = 1 << pr.log2ceil(N)
    pad = lambda X: [x for i in range(L * M) for x in X[i * N:(i + 1) * N] + [0] * (Np - N)]
    nv = pr.log2ceil(L * M * N)
    u = [rng.randrange(R) for _ in range(nv)]
    v = [rng.randrange(R) for _ in range(nv)]
    claim = _mle(pad([x * y % R for x, y in zip(A, B)]), u)
    want = pr.prove_elemul(A, B, L, M, N, u, v, claim)
    got = host.prove_elemul(gctx, gctx.fr_upload(A), gctx.fr_upload(B), L, M, N, u, v, claim)
    assert got[:3] == want[:3]
    assert got[3] == _pad4(want[3])


@pytest.mark.parametrize("nv,k", [(4, 3), (1, 1), (7, 2), (10, 4)])
def test_combine_claims(gctx, nv, k):
    from grape_b200 import host
    rng = random.Random(nv * 10 + k)
    size = 1 << nv
    X = [rng.randrange(R) for _ in range(size)]
    us = [[rng.randrange(R) for _ in range(nv)] for _ in range(k)]
    v = [rng.randrange(R) for _ in range(nv)]
    claims = [_mle(X, uj) for uj in us]
    want_ret, want_tr = pr.combine_claims(X, claims, us, v, size)
    got_ret, got_tr = host.combine_claims(gctx, gctx.fr_upload(X), size, claims, us, v)
    assert got_ret == want_ret == _mle(X, v)
    assert got_tr == _pad4(want_tr)


@pytest.mark.parametrize("L,N,M,K,P", [(1, 4, 8, 8, 2), (2, 4, 2, 24, 4), (4, 2, 4, 88, 8), (1, 16, 8, 2048, 8), (1, 3, 8, 44, 4), (2, 2, 2, 8, 8)])
def test_sharded_prove_matmul_equals_unsharded(gctx, L, N, M, K, P):
    """The inner dimension dealt to P provers by residue class.  The provers run one after another on
    this GPU (their kernels never wait on each other); their buffers are concatenated in rank order
    in place of the all-gather.  Claims and transcript must equal the single-prover proof bit for bit."""
    import numpy as np
    import grape_b200 as g
    from grape_b200 import host
    rng = random.Random(L * 1000 + N * 100 + M * 10 + K + P)
    draw = bn254.SplitMix64(K + P, 5)
    A = [rng.randrange(-2**15, 2**15) % R for _ in range(L * N * K)]
    B = [rng.randrange(-2**15, 2**15) % R for _ in range(L * M * K)]
    u = draw.fr_vec(pr.log2ceil(L * N * M))
    v = draw.fr_vec(pr.log2ceil(L * K))
    a_ = pr.partial_eval(list(A), len(A), u, N, pr.log2ceil(M), K)
    b_ = pr.partial_eval(list(B), len(B), u, M, 0, K)
    lL, u_end = pr.log2ceil(L), pr.log2ceil(L * N * M)
    w = pr.eq_weights(u[u_end - lL:u_end], lL, L)
    claim = sum(w[l] * a_[l * K + k] * b_[l * K + k] for l in range(L) for k in range(K)) % R
    single = host.prove_matmul(gctx, gctx.fr_upload(A), gctx.fr_upload(B), L, N, M, K, u, v, claim)
    want = pr.prove_matmul(A, B, L, N, M, K, u, v, claim)
    assert single[:3] == want[:3] and single[3] == _pad4(want[3])

    lp = P.bit_length() - 1
    n_el = host.matmul_partial_elems(L, K // P)
    gathered = gctx.alloc(P * n_el * 32)
    Aenc = host.encode_field(A)
    Benc = host.encode_field(B)
    for r in range(P):
        As = np.ascontiguousarray(Aenc.reshape(-1, K, 8)[:, r::P, :])
        Bs = np.ascontiguousarray(Benc.reshape(-1, K, 8)[:, r::P, :])
        rounds = host.prove_matmul_partial(gctx, gctx.upload(As), gctx.upload(Bs), L, N, M, K // P, u, v[lp:],
                                           gathered.at(r * n_el * 32))
        assert 3 * rounds + 2 == n_el
    got = host.prove_matmul_finish(gctx, gathered, P, L, N, M, K, u, v, claim)
    assert got[:3] == single[:3] and got[3] == single[3]
    # the gathered partial sums are the oracle's
    raw = gctx.download(gathered, P * n_el * 32).tobytes()
    for r in range(P):
        Asl = [A[(l * N + n) * K + k] for l in range(L) for n in range(N) for k in range(r, K, P)]
        Bsl = [B[(l * M + m) * K + k] for l in range(L) for m in range(M) for k in range(r, K, P)]
        sums, fa, fb = pr.prove_matmul_partial(Asl, Bsl, L, N, M, K // P, u, v[lp:])
        vals = bn254.fr_vec_from_bytes(raw[r * n_el * 32:(r + 1) * n_el * 32])
        assert vals == [x for q3 in sums for x in q3] + [fa, fb]
    # a wrong claim fails the round check
    with pytest.raises(g.GrapeError) as e:
        host.prove_matmul_finish(gctx, gathered, P, L, N, M, K, u, v, (claim + 1) % R)
    assert e.value.code == 3


def test_prove_matmul_mid_size_equals_c_oracle(gctx):
    """256 x 2048 . 512 x 2048 (1.5 M elements): the GPU proof from Fr tensors and from int32 tensors
    against the C restatement -- claims and every round polynomial."""
    import numpy as np
    from grape_b200 import host
    from oracle import cport
    rng = np.random.default_rng(5)
    N, M, K = 256, 512, 2048
    A = rng.integers(-2**15, 2**15, size=N * K).astype(np.int32)
    B = rng.integers(-2**15, 2**15, size=M * K).astype(np.int32)
    gctx.seed(15)
    u = host.decode_field(gctx.random_fr(pr.log2ceil(N * M)))
    v = host.decode_field(gctx.random_fr(pr.log2ceil(K)))
    dAi, dBi = gctx.upload(A), gctx.upload(B)
    dA, dB = gctx.alloc(N * K * 32), gctx.alloc(M * K * 32)
    gctx.fr_from_i32(dAi, N * K, dA)
    gctx.fr_from_i32(dBi, M * K, dB)
    # the claim: <fold(A), fold(B)>, by the library's own fold and sum
    du = gctx.fr_upload(u)
    a_, b_, one = gctx.alloc(K * 32), gctx.alloc(K * 32), gctx.alloc(32)
    gctx.fr_fold(dA, N * K, du.at(pr.log2ceil(M) * 32), N, K, a_)
    gctx.fr_fold(dB, M * K, du, M, K, b_)
    gctx.fr_binary("mul", a_, b_, a_, K)
    gctx.fr_sum(a_, K, one)
    claim = gctx.fr_download(one, 1)[0]
    got_i = host.prove_matmul_i32(gctx, dAi, dBi, 1, N, M, K, u, v, claim)
    got = host.prove_matmul(gctx, dA, dB, 1, N, M, K, u, v, claim)
    assert got == got_i
    rc, ca, cb, cfinal, ctr = cport.prove_matmul_l1(A, B, N, M, K, host.encode_field(u), host.encode_field(v),
                                                    host.encode_field([claim]))
    assert rc == 0
    dec = lambda x: host.decode_field(x.reshape(-1, 8))
    assert (dec(ca)[0], dec(cb)[0], dec(cfinal)[0]) == got[:3]
    assert [dec(ctr[i]) for i in range(ctr.shape[0])] == [p[:3] for p in got[3]]
