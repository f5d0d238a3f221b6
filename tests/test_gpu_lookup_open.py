"""Parity of the lookup argument and of the Hyrax opening with the oracle (claims, round
polynomials, multiplicities, tables, proof elements), with the prover randomness seeded identically."""
import random

import numpy as np
import pytest

from oracle import bn254, cport
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def test_lookup_range_power_of_two(gctx):
    from grape_b200 import host
    rng = random.Random(1)
    gctx.seed(77)
    draw = bn254.SplitMix64(77)
    lk = host.Lookup(gctx, -8, 16)
    ref = pr.LookupRange(-8, 16, draw.next_fr())
    assert lk.alpha == ref.alpha and lk.beta == ref.beta and lk.n == 16
    assert lk.table("T") == ref.T and lk.table("B") == ref.B
    D = 256
    S = [rng.randrange(-8, 8) % R for _ in range(D)]
    v = [rng.randrange(R) for _ in range(8)]
    u = draw.fr_vec(8)
    want = ref.prove(S, v, u)
    dS, dA = gctx.fr_upload(S), gctx.alloc(D * 32)
    claim, tr = lk.prove(dS, D, dA, v)
    assert claim == want["claim"] == _mle(S, v)
    assert tr == want["transcript"]
    assert lk.table("m") == want["m"]
    lk.close()


def test_lookup_range_padded_rows(gctx):
    """D is not a power of two: rows of 6 padded to 8, pad count lands in the bin of value zero."""
    from grape_b200 import host
    rng = random.Random(2)
    gctx.seed(5)
    draw = bn254.SplitMix64(5)
    lk = host.Lookup(gctx, -4, 8)
    ref = pr.LookupRange(-4, 8, draw.next_fr())
    rows, inner, inner_pad = 4, 6, 8
    D = rows * inner
    S = [rng.randrange(-4, 4) % R for _ in range(D)]
    v = [rng.randrange(R) for _ in range(5)]
    u = draw.fr_vec(5)
    want = ref.prove(S, v, u, inner=inner, inner_pad=inner_pad)
    dS = gctx.alloc(32 * 32)
    s_enc = host.encode_field(S)    # keep the host array alive across the copy
    gctx._check(gctx.lib.grape_h2d(gctx.handle, dS.ptr, s_enc.ctypes.data, D * 32))
    gctx.sync()
    gctx.sync()
    dA = gctx.alloc(32 * 32)
    claim, tr = lk.prove(dS, D, dA, v, inner=inner, inner_pad=inner_pad)
    assert claim == want["claim"] and tr == want["transcript"]
    assert lk.table("m") == want["m"] and sum(want["m"]) == 32
    lk.close()


def test_lookup_with_commitments(gctx):
    """The commitments to A = 1/(S+beta) and to the multiplicities, as the reference forms them."""
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    rng = random.Random(3)
    gens = wl.make_generators(gctx, 512, seed=31)
    table = g.GeneratorTable(gctx, gens, 8, 1)
    ctable = cport.table_build(gens)
    gctx.seed(9)
    draw = bn254.SplitMix64(9)
    lk = host.Lookup(gctx, -512, 1024)
    ref = pr.LookupRange(-512, 1024, draw.next_fr())
    D, msm = 4096, 16
    S = [rng.randrange(-512, 512) % R for _ in range(D)]
    v = [rng.randrange(R) for _ in range(12)]
    u = draw.fr_vec(12)
    want = ref.prove(S, v, u)
    dS, dA = gctx.fr_upload(S), gctx.alloc(D * 32)
    comA, comm = gctx.alloc(D // (msm * 16) * 96), gctx.alloc(1024 // 512 * 96)
    claim, tr = lk.prove(dS, D, dA, v, table=table, msm_size=msm, d_com_A=comA, d_com_m=comm)
    assert claim == want["claim"] and tr == want["transcript"]
    wantA = cport.commit_fr(host.encode_field(want["A"]), msm * 16, ctable)
    wantm = cport.commit_fr(host.encode_field(want["m"]), 512, ctable)
    assert gctx.download(comA, wantA.nbytes).tobytes() == wantA.tobytes()
    assert gctx.download(comm, wantm.nbytes).tobytes() == wantm.tobytes()
    lk.close()
    table.close()


def test_lookup_mapping(gctx):
    from grape_b200 import host
    rng = random.Random(4)
    gctx.seed(13)
    draw = bn254.SplitMix64(13)
    mp = [rng.randrange(-1000, 1000) for _ in range(32)]
    lk = host.Lookup(gctx, -16, 32, np.array(mp, dtype=np.int32))
    ref = pr.LookupRangeMapping(-16, 32, mp, draw.next_fr(), draw.next_fr())
    assert lk.r == ref.r and lk.table("T") == ref.T and lk.table("B") == ref.B
    D = 128
    s_in = [rng.randrange(-16, 16) for _ in range(D)]
    s_out = [mp[s + 16] for s in s_in]
    v = [rng.randrange(R) for _ in range(7)]
    u = draw.fr_vec(7)
    want = ref.prove_pairs([s % R for s in s_in], [s % R for s in s_out], v, u)
    d_in, d_out = gctx.fr_upload(s_in), gctx.fr_upload(s_out)
    work, dA = gctx.alloc(D * 32), gctx.alloc(D * 32)
    claim, tr = lk.prove_pairs(d_in, d_out, D, work, dA, v)
    assert claim == want["claim"] and tr == want["transcript"] and lk.table("m") == want["m"]
    lk.close()


def test_lookup_rejects_query_outside_table(gctx):
    import grape_b200 as g
    from grape_b200 import host
    lk = host.Lookup(gctx, -8, 16)
    S = [3 % R] * 63 + [100]
    with pytest.raises(g.GrapeError) as e:
        lk.prove(gctx.fr_upload(S), 64, gctx.alloc(64 * 32), [5, 6, 7, 8, 9, 10])
    assert e.value.code == 3
    lk.close()


@pytest.mark.parametrize("layer_num,N,rows", [(2, 2, 2), (1, 3, 4), (4, 1, 1)])
def test_hyrax_open_and_verify(gctx, layer_num, N, rows):
    import grape_b200 as g
    from grape_b200 import host
    rng = random.Random(layer_num * 10 + N)
    wd = N * 16
    new_n = (1 << pr.log2ceil(N)) * 16
    gens = bn254.make_generators(new_n, seed=41)
    gj = g.encode_jacobian(gens)
    table = g.GeneratorTable(gctx, gj, 8, 1)
    size = layer_num * rows * wd
    t = [rng.randrange(-2**15, 2**15) for _ in range(size)]
    # the tensor is committed in its padded layout (every N-chunk padded to a power of two), which is
    # what the reference does before commit (pad_int, test/commit.cu:63-64)
    pad_n = new_n // 16
    d_int = gctx.upload(np.array(t, dtype=np.int32))
    n_pad = (size // N) * pad_n
    d_pad = gctx.alloc(n_pad * 4)
    gctx.pad_i32(d_int, d_pad, N, pad_n, n_pad)
    t_pad = [int(x) for x in gctx.download(d_pad, n_pad * 4, dtype=np.int32)]
    assert t_pad == [t[(i // pad_n) * N + i % pad_n] if i % pad_n < N else 0 for i in range(n_pad)]
    com = gctx.alloc((n_pad // new_n) * 96)
    g.commit_i32(gctx, table, d_pad, n_pad, new_n, com)
    commitments = g.decode_jacobian(gctx.download(com, (n_pad // new_n) * 96).reshape(-1, 24))
    assert commitments == pr.commit_rows(t_pad, new_n, gens)
    e = [rng.randrange(R) for _ in range(pr.log2ceil(size))]
    c = rng.randrange(R)
    gctx.seed(1234)
    d = bn254.SplitMix64(1234).fr_vec(new_n)
    tf = [x % R for x in t]
    want = pr.hyrax_open(tf, e, c, size, N, layer_num, gens, gens[0], d)
    d_t = gctx.fr_upload(tf)
    got = host.hyrax_open(gctx, table, d_t, size, N, layer_num, e, c, gj[0])
    assert got["result"] == want["result"]
    assert got["z"] == want["z"]
    assert got["com_d"] == want["com_d"] and got["com_ad"] == want["com_ad"]
    assert gctx.fr_download(d_t, size) == tf  # the tensor is left intact
    proof = {"result": got["result"], "z": got["z"], "com_d": got["com_d"], "com_ad": got["com_ad"]}
    assert pr.hyrax_verify(commitments, proof, e, c, size, N, layer_num, gens, gens[0])
    table.close()


@pytest.mark.parametrize("inner,inner_pad,window_bits,affine", [(11, 16, 8, False), (6, 8, 13, False), (24, 32, 16, False),
                                                                  (11, 16, 8, True), (6, 8, 13, True)])
def test_lookup_commitment_of_padded_rows(gctx, inner, inner_pad, window_bits, affine):
    """Rows padded inner -> inner_pad: the padded columns of A all hold 1 / (pad + beta).  The prover
    commits them through one shared point instead of one addition per column and window; the row
    commitments must still equal a plain commitment of the padded A.  With `affine` the accumulation is
    forced onto the affine-accumulator kernel, which walks the same skipped columns."""
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    rng = random.Random(inner * 10 + window_bits)
    rows_in = 256                       # sub-rows of `inner` values
    D = rows_in * inner
    Dp = rows_in * inner_pad            # a power of two
    msm = 2 * inner_pad // 16 * 4       # row of msm * 16 generators = 8 sub-rows
    wd = msm * 16
    gens = wl.make_generators(gctx, max(wd, 256), seed=inner)   # the multiplicities are committed over 256
    table = g.GeneratorTable(gctx, gens, window_bits, 1)
    ctable = cport.table_build(gens)
    gctx.seed(21)
    draw = bn254.SplitMix64(21)
    lk = host.Lookup(gctx, -128, 256)
    ref = pr.LookupRange(-128, 256, draw.next_fr())
    S = [rng.randrange(-128, 128) % R for _ in range(D)]
    v = [rng.randrange(R) for _ in range(pr.log2ceil(Dp))]
    u = draw.fr_vec(pr.log2ceil(Dp))
    want = ref.prove(S, v, u, inner=inner, inner_pad=inner_pad)
    assert len(want["A"]) == Dp
    dS, dA = gctx.alloc(Dp * 32), gctx.alloc(Dp * 32)
    s_enc = host.encode_field(S)    # keep the host array alive across the copy
    gctx._check(gctx.lib.grape_h2d(gctx.handle, dS.ptr, s_enc.ctypes.data, D * 32))
    gctx.sync()
    comA = gctx.alloc(Dp // wd * 96)
    try:
        if affine:
            gctx.set_affine_commit(2, 8, 1)
        claim, tr = lk.prove(dS, D, dA, v, inner=inner, inner_pad=inner_pad, table=table, msm_size=msm, d_com_A=comA)
    finally:
        gctx.set_affine_commit(-1)
    assert claim == want["claim"] and tr == want["transcript"]
    wantA = cport.commit_fr(host.encode_field(want["A"]), wd, ctable)
    assert gctx.download(comA, wantA.nbytes).tobytes() == wantA.tobytes()
    # and equals the plain commitment of the same padded tensor by this library
    plain = gctx.alloc(Dp // wd * 96)
    g.commit_fr(gctx, table, gctx.fr_upload(want["A"]), Dp, wd, plain)
    assert gctx.download(plain, wantA.nbytes).tobytes() == wantA.tobytes()
    lk.close()
    table.close()


def _lookup_commitment(gctx, lk, S_enc, D, Dp, v, table, msm, wd, inner, inner_pad, mode, seed):
    """One range-lookup proof with the A-commitment path forced to `mode`; returns (claim, com_A bytes, A bytes)."""
    gctx.set_bucket_commit(mode)
    gctx.seed(seed)
    dS, dA = gctx.alloc(Dp * 32), gctx.alloc(Dp * 32)
    gctx._check(gctx.lib.grape_h2d(gctx.handle, dS.ptr, S_enc.ctypes.data, D * 32))
    gctx.sync()
    comA = gctx.alloc(Dp // wd * 96)
    kw = dict(inner=inner, inner_pad=inner_pad) if inner else {}
    l0 = gctx.launches
    claim, tr = lk.prove(dS, D, dA, v, table=table, msm_size=msm, d_com_A=comA, **kw)
    out = (claim, tr, gctx.download(comA, Dp // wd * 96).tobytes(), gctx.launches - l0)
    gctx.set_bucket_commit(1)
    return out


@pytest.mark.parametrize("n_table,rows_in,inner,inner_pad,msm,window_bits,skew", [
    (256, 4096, 0, 0, 64, 8, False),        # 4 rows of 1024 elements over a 256-entry table
    (256, 512, 11, 16, 32, 13, False),      # padded rows: the padded columns go through the shared point
    (256, 2048, 0, 0, 128, 8, True),        # one value taken by half of the elements, many entries unused
    (65536, 1 << 18, 0, 0, 1 << 13, 8, False),  # a table wider than one block's counters: two sort parts
])
def test_bucket_commitment_equals_direct_commitment(gctx, n_table, rows_in, inner, inner_pad, msm, window_bits, skew):
    """A committed by the bucket method (generators summed per table entry, then one variable-base
    multi-scalar multiplication per row) gives byte-identical commitments, claims and transcripts."""
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    rng = np.random.default_rng(n_table + rows_in)
    low = -(n_table // 2)
    if inner:
        D, Dp = rows_in * inner, rows_in * inner_pad
    else:
        D = Dp = rows_in
    wd = msm * 16
    vals = rng.integers(low, low + n_table, size=D)
    if skew:
        vals[rng.random(D) < 0.5] = low + 3
        vals[(vals > low + 20) & (vals < low + 40)] = low + 50
    S_enc = host.encode_field([int(x) for x in vals]) if D <= 1 << 16 else None
    if S_enc is None:   # large case: build the field encoding on the GPU
        d_int = gctx.upload(vals.astype(np.int32))
        d_fr = gctx.alloc(D * 32)
        gctx.fr_from_i32(d_int, D, d_fr)
        S_enc = gctx.download(d_fr, D * 32).reshape(D, 8)
    gens = wl.make_generators(gctx, max(wd, 4096), seed=n_table)
    table = g.GeneratorTable(gctx, gens, window_bits, 1)
    v = [int(x) for x in rng.integers(1, 2**62, size=pr.log2ceil(Dp))]
    results = []
    for mode in (0, 2):
        gctx.seed(77)
        lk = host.Lookup(gctx, low, n_table)
        results.append(_lookup_commitment(gctx, lk, S_enc, D, Dp, v, table, msm, wd, inner, inner_pad, mode, seed=78))
        lk.close()
    assert results[0][0] == results[1][0] and results[0][1] == results[1][1]
    assert results[0][2] == results[1][2]
    assert results[0][3] != results[1][3]   # the two modes really took different kernel sequences
    if D <= 1 << 13:    # and both equal the C oracle's commitment of A = 1/(S + beta)
        ctable = cport.table_build(gens)
        gctx.seed(77)
        draw = bn254.SplitMix64(77)
        ref = pr.LookupRange(low, n_table, draw.next_fr())
        draw2 = bn254.SplitMix64(78)
        kw = dict(inner=inner, inner_pad=inner_pad) if inner else {}
        want = ref.prove([int(x) % R for x in vals], v, draw2.fr_vec(pr.log2ceil(Dp)), **kw)
        wantA = cport.commit_fr(host.encode_field(want["A"]), wd, ctable)
        assert results[1][2] == wantA.tobytes()
    table.close()


def test_lookup_mid_size_equals_c_oracle(gctx):
    """2^18 queries into a 2^12-entry table: multiplicities, claim and every round polynomial against
    the C restatement of tLookupRange::prove."""
    from grape_b200 import host
    D, N, low = 1 << 18, 1 << 12, -(1 << 11)
    rng = np.random.default_rng(18)
    q = rng.integers(low, low + N, size=D).astype(np.int32)
    gctx.seed(40)
    lk = host.Lookup(gctx, low, N)
    v = host.decode_field(gctx.random_fr(18))
    gctx.seed(41)
    u_enc = gctx.random_fr(18)     # what the prover draws inside the call below
    gctx.seed(41)
    dS = gctx.alloc(D * 32)
    gctx.fr_from_i32(gctx.upload(q), D, dS)
    claim, tr = lk.prove(dS, D, gctx.alloc(D * 32), v)
    rc, m, s_claim, final, ctr = cport.lookup_range(q, low, N, host.encode_field([lk.alpha])[0], u_enc, host.encode_field(v))
    assert rc == 0
    assert [int(x) for x in m] == lk.table("m")
    assert host.decode_field(s_claim.reshape(1, 8))[0] == claim
    assert [host.decode_field(ctr[i]) for i in range(ctr.shape[0])] == tr
    lk.close()


def test_open_of_row_blocks_equals_open_of_the_whole_tensor(gctx):
    """The identity behind ``parallel.hyrax_open_sharded``: folding every block of rows over the low row
    variables, then the stacked partial vectors over the high ones, then opening the single row, gives
    the proof of the unsharded opening (here the four blocks are folded one after the other on one GPU)."""
    import random
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    rnd = random.Random(31)
    N, rows, P = 4, 16, 4
    wd = N * 16
    gens_j = wl.make_generators(gctx, wd, seed=8)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    t = [rnd.randrange(R) for _ in range(rows * wd)]
    e = [rnd.randrange(R) for _ in range(pr.log2ceil(rows * wd))]
    c = rnd.randrange(R)
    gctx.seed(77)
    whole = host.hyrax_open(gctx, table, gctx.fr_upload(t), rows * wd, N, 1, e, c, gens_j[0])
    lw, block = pr.log2ceil(wd), rows // P
    d_e = gctx.fr_upload(e)
    d_all = gctx.alloc(P * wd * 32)
    for r in range(P):
        d_blk = gctx.fr_upload(t[r * block * wd:(r + 1) * block * wd])
        gctx.fr_fold(d_blk, block * wd, d_e.at(lw * 32), block, wd, d_all.at(r * wd * 32))
    d_x = gctx.alloc(wd * 32)
    gctx.fr_fold(d_all, P * wd, d_e.at((lw + pr.log2ceil(block)) * 32), P, wd, d_x)
    gctx.seed(77)
    shard = host.hyrax_open(gctx, table, d_x, wd, N, 1, e[:lw], c, gens_j[0])
    assert shard["result"] == whole["result"] == pr.partial_eval(list(t), rows * wd, e, rows * wd, 0, 1)[0]
    assert shard.z_raw.tobytes() == whole.z_raw.tobytes() and shard.com_raw.tobytes() == whole.com_raw.tobytes()
    table.close()
