"""Parity at the sizes the benchmark configurations name, against the C restatement of the reference
(oracle/grape_oracle.c through oracle/cport.py; it finishes each case in well under a minute on the
host cores):

  C1  Hyrax::commit(int*) of a 1024 x 1024 int16 tensor over 1024 generators   (test/commit.cu:39-61)
  C2  prove_matmul, A 2048 x 4096 . B 4096 x 4096                               (test/matmul.cu:65-105)
  C3  tLookupRange::prove, 2^22 queries into a 2^16 table, with commitments     (test/tlookupTest.cu:40-59)
  C4  one LLaMA-2-7B-shaped layer's 49 408 rows over 4096 generators, sampled rows
  C5  the feed-forward half of the layer driver at tokens 256, dim 512 against the Python oracle walk
"""
import numpy as np
import pytest

from oracle import bn254, cport

pytestmark = pytest.mark.gpu
R = bn254.R


def _normal_i32(rng, n, lo, hi):
    from grape_b200 import workloads as wl
    return wl.quantised_normal(rng, n, lo=lo, hi=hi)


@pytest.mark.parametrize("window_bits,n_windows", [(16, 1), (8, 2)])
def test_c1_commit_1024x1024_int16(gctx, window_bits, n_windows):
    import grape_b200 as g
    from grape_b200 import workloads as wl
    wd = rows = 1024
    gens = wl.make_generators(gctx, wd, 0xC1)
    table = g.GeneratorTable(gctx, gens, window_bits, n_windows)
    rng = np.random.default_rng(0xC1)
    s = rng.integers(-(1 << 15), 1 << 15, size=rows * wd).astype(np.int32)
    d, out = gctx.upload(s), gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, d, s.size, wd, out, max_bits=16)
    got = gctx.download(out, rows * 96).reshape(rows, 24)
    assert gctx.status() == 0
    want = cport.commit_i32(s, wd, cport.table_build(gens))
    assert np.array_equal(got, want)
    # the host-buffer entry point returns the same records
    got_h = g.commit_i32_host(gctx, table, s, wd, max_bits=16)
    assert np.array_equal(got_h, want)
    table.close()


def test_c2_prove_matmul_2048x4096x4096(gctx):
    from grape_b200 import host
    L, N, M, K = 1, 2048, 4096, 4096
    rng = np.random.default_rng(0xC2)
    A = _normal_i32(rng, N * K, -2**31, 2**31 - 1)
    B = _normal_i32(rng, M * K, -2**31, 2**31 - 1)
    dAi, dBi = gctx.upload(A), gctx.upload(B)
    dA, dB = gctx.alloc(N * K * 32), gctx.alloc(M * K * 32)
    gctx.seed(0xC2)
    lM, lN, lK = 12, 11, 12
    u = host.decode_field(gctx.random_fr(lM + lN))
    v = host.decode_field(gctx.random_fr(lK))
    # the claim Y~(u) = sum_k A~(u_N, k) B~(u_M, k), formed with the library's folds
    du = gctx.fr_upload(u)
    a_, b_, one = gctx.alloc(K * 32), gctx.alloc(K * 32), gctx.alloc(32)
    gctx.fr_from_i32(dAi, N * K, dA)
    gctx.fr_from_i32(dBi, M * K, dB)
    gctx.fr_fold(dA, N * K, du.at(lM * 32), N, K, a_)
    gctx.fr_fold(dB, M * K, du, M, K, b_)
    gctx.fr_binary("mul", a_, b_, a_, K)
    gctx.fr_sum(a_, K, one)
    claim = gctx.fr_download(one, 1)[0]
    got = host.prove_matmul(gctx, dA, dB, L, N, M, K, u, v, claim)
    got_i = host.prove_matmul_i32(gctx, dAi, dBi, L, N, M, K, u, v, claim)
    assert got_i == got
    enc = host.encode_field
    rc, ca, cb, cfinal, ctr = cport.prove_matmul_l1(A, B, N, M, K, enc(u), enc(v), enc([claim]))
    assert rc == 0          # every round check of the restatement closes on this claim
    dec = lambda rec: host.decode_field(np.asarray(rec).reshape(1, 8))[0]
    assert (dec(ca), dec(cb), dec(cfinal)) == (got[0], got[1], got[2])
    assert [host.decode_field(ctr[i]) for i in range(ctr.shape[0])] == [p[:3] for p in got[3]]
    assert len(got[3]) == lK
    for b in (dAi, dBi, dA, dB):
        b.free()


def test_c3_range_lookup_2p22_queries(gctx):
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    D, Nt, low, wd = 1 << 22, 1 << 16, -(1 << 15), 4096
    rng = np.random.default_rng(0xC3)
    q = rng.integers(low, low + Nt, size=D).astype(np.int32)
    q[:4] = [low, low + Nt - 1, 0, -1]
    gens = wl.make_generators(gctx, wd, 0xC3)
    table = g.GeneratorTable(gctx, gens, 13, 1)
    dqi, dS, dA = gctx.upload(q), gctx.alloc(D * 32), gctx.alloc(D * 32)
    m_wd = 256 * 16    # the multiplicities are committed in rows of 2^(log2(N)/2) * 16 elements (src/tlookup.cu:321)
    com_A, com_m = gctx.alloc(D // wd * 96), gctx.alloc(Nt // m_wd * 96)
    gctx.seed(0xC3)
    lk = host.Lookup(gctx, low, Nt)
    vv = host.decode_field(gctx.random_fr(22))
    gctx.seed(0xC33)
    u_enc = gctx.random_fr(22)            # what the prover draws inside the next call
    gctx.seed(0xC33)
    gctx.fr_from_i32(dqi, D, dS)
    claim, tr = lk.prove(dS, D, dA, vv, table=table, msm_size=256, d_com_A=com_A, d_com_m=com_m)
    m = lk.table("m")
    rc, c_m, c_claim, c_final, c_tr = cport.lookup_range(q, low, Nt, host.encode_field([lk.alpha])[0], u_enc,
                                                         host.encode_field(vv))
    assert rc == 0
    assert [int(x) for x in c_m] == m                        # multiplicities
    assert int(np.sum(c_m)) == D
    assert host.decode_field(c_claim.reshape(1, 8))[0] == claim
    assert [host.decode_field(c_tr[i]) for i in range(c_tr.shape[0])] == tr   # every round polynomial
    # the commitments of sampled rows of A = 1 / (S + beta) (rebuilt on the host: the prover folds its A in
    # place) and of every row of m
    ctable = cport.table_build(gens)
    beta = lk.beta
    got_A = gctx.download(com_A, D // wd * 96).reshape(-1, 24)
    inv_of = {}
    for r in (0, 1, 511, 1023):
        row = [inv_of.setdefault(int(x), pow((int(x) + beta) % R, -1, R)) for x in q[r * wd:(r + 1) * wd]]
        assert np.array_equal(cport.commit_fr(host.encode_field(row), wd, ctable)[0], got_A[r])
    m_enc = host.encode_field(m)
    got_m = gctx.download(com_m, Nt // m_wd * 96).reshape(-1, 24)
    want_m = cport.commit_fr(m_enc, m_wd, ctable)
    assert np.array_equal(got_m, want_m)
    # the same lookup with the bucket method for A commits to the same rows
    gctx.set_bucket_commit(2)
    try:
        gctx.seed(0xC33)
        gctx.fr_from_i32(dqi, D, dS)
        com_A2 = gctx.alloc(D // wd * 96)
        claim2, tr2 = lk.prove(dS, D, dA, vv, table=table, msm_size=256, d_com_A=com_A2, d_com_m=com_m)
        assert (claim2, tr2) == (claim, tr)
        assert np.array_equal(gctx.download(com_A2, D // wd * 96).reshape(-1, 24), got_A)
    finally:
        gctx.set_bucket_commit(1)
    table.close()
    for b in (dqi, dS, dA):
        b.free()


def test_c4_layer_rows_sampled(gctx):
    import grape_b200 as g
    from grape_b200 import workloads as wl
    wd = 4096
    n = wl.layer_weight_elements()
    rows = n // wd
    assert rows == 49408
    gens = wl.make_generators(gctx, wd, 0xC4)
    table = g.GeneratorTable(gctx, gens, 16, 1)
    rng = np.random.default_rng(0xC4)
    s = wl.quantised_normal(rng, n)
    d, out = gctx.upload(s), gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, d, n, wd, out, max_bits=16)
    got = gctx.download(out, rows * 96).reshape(rows, 24)
    assert gctx.status() == 0
    ctable = cport.table_build(gens)
    for r0 in (0, 4096, 16383, 30000, 49408 - 64):
        assert np.array_equal(cport.commit_i32(s, wd, ctable, r0, r0 + 64), got[r0:r0 + 64])
    # linearity over the whole tensor: the commitments of s and of -s are opposite points, row by row
    neg = gctx.upload(-s)
    out2 = gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, neg, n, wd, out2, max_bits=16)
    got2 = gctx.download(out2, rows * 96).reshape(rows, 24)
    P = bn254.P
    x1 = got[:, :8]; x2 = got2[:, :8]
    assert np.array_equal(x1, x2)                      # same x
    ys = g.decode_field(got[::997, 8:16].copy(), P)
    ys2 = g.decode_field(got2[::997, 8:16].copy(), P)
    assert all((a + b) % P == 0 for a, b in zip(ys, ys2))
    table.close()
    for b in (d, out, neg, out2):
        b.free()


def test_c5_ffn_block_tokens256_dim512_matches_oracle(gctx):
    """The feed-forward half of the layer driver (test/llm.cu:73-239) at tokens 256, dim 512, ffn 1376
    (padded to 2048): every junction value equals the Python oracle's walk with the same random stream."""
    import grape_b200 as g
    from grape_b200 import layer, workloads as wl
    from oracle import layer as olayer
    shape = layer.FFNShape(layer_num=1, tokens=256, dim=512, ffn=1376, scale1=256, scale2=512, swiglu_low=-256,
                           swiglu_len=512, npoints=64)
    t = layer.synthesize_ffn(shape, seed=11, x_range=16, w_std=2.0)
    assert t["gate_q"].min() >= -256 and t["gate_q"].max() < 256
    gens_j = wl.make_generators(gctx, shape.ffn_pad * 16, seed=77)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    gctx.seed(2025)
    prover = layer.FFNProver(gctx, shape, table, gens_j[0], t["swiglu_table"])
    trace = prover.prove(t)
    gens = g.decode_jacobian(gens_j)
    ctable = cport.table_build(gens_j)

    def msm_fn(scalars, points):
        enc = np.frombuffer(bn254.fr_vec_to_bytes(scalars), dtype=np.uint32).reshape(-1, 8)
        rec = cport.commit_fr(enc, len(scalars), ctable[:, :len(scalars)].copy())
        return bn254.jacobian_from_bytes(rec[0].tobytes())

    flat = {k: v.reshape(-1).tolist() for k, v in t.items()}
    want = olayer.prove_ffn(flat, shape, gens, bn254.SplitMix64(2025), msm_fn)
    for key in ("skip", "down_out", "upSilu", "silu_at_e2", "up_out", "gate_out", "normOutSecond",
                "normOutSecond_point", "skip_point"):
        assert trace.values[key] == want[key], key
    prover.release_pool()
    table.close()
