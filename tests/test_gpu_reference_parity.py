"""Pins the oracle AND this library against the reference's own code.

``oracle/_ref/ref_harness`` is the reference's unmodified src/*.cu linked with a libff stand-in
(oracle/ref_shim) and built by ``make -C oracle ref`` where the reference tree is available.  The
harness runs the reference's commit (int and Fr), open, prove_matmul, prove_eleMul, combine_claims,
tLookupRange::prove and tLookupRangeMapping::prove on a blob of inputs with a seeded random stream; here the same inputs and the same stream go through
the oracle and through libgrape_b200, and every value is compared.  Shapes respect what the
reference's unguarded kernels can take (row counts that fill whole blocks, power-of-two sizes).
"""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
HARNESS = ROOT / "oracle" / "_ref" / "ref_harness"
R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


@pytest.mark.skipif(not HARNESS.exists(), reason="reference build (oracle/_ref) not present")
def test_reference_outputs_equal_oracle_and_library(gctx, tmp_path):
    import grape_b200 as g
    from grape_b200 import host, workloads as wl
    n_gens, N, layer_num = 1024, 4, 2
    size = 64 * N * 16                      # 64 rows: whole blocks for the reference's reduce kernel
    L, Nn, M, K = 1, 4, 8, 6
    lk_len, lk_D = 4096, 16384
    rng = np.random.default_rng(23)
    tensor = rng.integers(-2**31, 2**31, size=size, dtype=np.int64).astype(np.int32)
    A = rng.integers(-2**12, 2**12, size=L * Nn * K).astype(np.int32)
    B = rng.integers(-2**12, 2**12, size=L * M * K).astype(np.int32)
    Y = (A.reshape(L, Nn, K).astype(np.int64) @ B.reshape(L, M, K).astype(np.int64).transpose(0, 2, 1)).astype(np.int32)
    Q = rng.integers(-(lk_len // 2), lk_len // 2, size=lk_D).astype(np.int32)
    eL, eM, eN = 2, 4, 8
    esize = eL * eM * eN
    EA = rng.integers(-2**20, 2**20, size=esize).astype(np.int32)
    EB = rng.integers(-2**20, 2**20, size=esize).astype(np.int32)
    map_len, map_D, map_low = 4096, 16384, -2048
    map_table = rng.integers(-2**16, 2**16, size=map_len).astype(np.int32)
    MIN = rng.integers(map_low, map_low + map_len, size=map_D).astype(np.int32)
    MOUT = map_table[MIN - map_low]
    blob, out = tmp_path / "in.bin", tmp_path / "out.bin"
    map_table.tofile(str(blob) + ".table")
    with open(blob, "wb") as f:
        f.write(np.array([n_gens, size, N, layer_num, L, Nn, M, K, lk_len, lk_D], dtype=np.uint32).tobytes())
        for arr in (tensor, A, B, Y, Q):
            f.write(arr.tobytes())
        f.write(np.array([eL, eM, eN, map_len, map_D, map_low & 0xFFFFFFFF], dtype=np.uint32).tobytes())
        for arr in (EA, EB, MIN, MOUT):
            f.write(arr.tobytes())
    env = dict(os.environ, OMP_NUM_THREADS="1")   # the reference draws the blinding vector in an OpenMP loop
    res = subprocess.run([str(HARNESS), "parity", str(blob), str(out)], capture_output=True, text=True, env=env,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    raw = out.read_bytes()
    pos = 0

    def take(n):
        nonlocal pos
        b = raw[pos:pos + n]
        pos += n
        return b

    wd = N * 16
    rows = size // wd
    # ---- the reference's values
    ref_gens = take(n_gens * 96)
    ref_c0 = bn254.jacobian_vec_from_bytes(take(rows * 96))
    ref_c1 = bn254.jacobian_vec_from_bytes(take(rows * 96))
    ref_result, ref_z = take(32), take(wd * 32)
    ref_com_d, ref_com_ad = bn254.jacobian_from_bytes(take(96)), bn254.jacobian_from_bytes(take(96))
    ref_claim0, ref_a, ref_b, ref_final = take(32), take(32), take(32), take(32)
    ref_lookup = take(32)
    ref_ecl0, ref_ea, ref_eb = take(32), take(32), take(32)
    ref_k1, ref_k2, ref_comb = take(32), take(32), take(32)
    ref_map_r, ref_map_val = take(32), take(32)
    assert pos == len(raw)

    # ---- the oracle, same stream
    draw = bn254.SplitMix64(99)
    gens = [bn254.scalar_mul(draw.next_fr(), bn254.G1_GEN) for _ in range(n_gens)]
    assert ref_gens == b"".join(bn254.jacobian_to_bytes(p) for p in gens)
    t_int = [int(x) for x in tensor]
    want_com = pr.commit_rows(t_int, wd, gens)
    assert ref_c0 == want_com and ref_c1 == want_com
    e = draw.fr_vec(pr.log2ceil(size))
    c = draw.next_fr()
    d = draw.fr_vec(wd)
    proof = pr.hyrax_open([x % R for x in t_int], e, c, size, N, layer_num, gens, gens[0], d)
    assert ref_result == bn254.fr_to_bytes(proof["result"])
    assert ref_z == bn254.fr_vec_to_bytes(proof["z"])
    assert ref_com_d == proof["com_d"] and ref_com_ad == proof["com_ad"]
    u = draw.fr_vec(pr.log2ceil(L * Nn * M))
    v = draw.fr_vec(pr.log2ceil(K * L))
    claim = _mle([int(x) % R for x in Y.reshape(-1)], u)
    a_cl, b_cl, final, _ = pr.prove_matmul([int(x) % R for x in A], [int(x) % R for x in B], L, Nn, M, K, u, v, claim)
    assert (ref_claim0, ref_a, ref_b, ref_final) == tuple(bn254.fr_to_bytes(x) for x in (claim, a_cl, b_cl, final))
    lk = pr.LookupRange(-(lk_len // 2), lk_len, draw.next_fr())
    lv = draw.fr_vec(pr.log2ceil(lk_D))
    lu = draw.fr_vec(pr.log2ceil(lk_D))
    got = lk.prove([int(x) % R for x in Q], lv, lu)
    assert ref_lookup == bn254.fr_to_bytes(got["claim"])
    fa, fb = [int(x) % R for x in EA], [int(x) % R for x in EB]
    eu, ev = draw.fr_vec(6), draw.fr_vec(6)
    ecl = _mle([x * y % R for x, y in zip(fa, fb)], eu)
    o_ea, o_eb, _, _ = pr.prove_elemul(fa, fb, eL, eM, eN, eu, ev, ecl)
    assert (ref_ecl0, ref_ea, ref_eb) == tuple(bn254.fr_to_bytes(x) for x in (ecl, o_ea, o_eb))
    u1, u2, cv = draw.fr_vec(6), draw.fr_vec(6), draw.fr_vec(6)
    k1, k2 = _mle(fa, u1), _mle(fa, u2)
    o_comb, _ = pr.combine_claims(fa, [k1, k2], [u1, u2], cv, esize)
    assert (ref_k1, ref_k2, ref_comb) == tuple(bn254.fr_to_bytes(x) for x in (k1, k2, o_comb))
    omap = pr.LookupRangeMapping(map_low, map_len, [int(x) for x in map_table], draw.next_fr(), draw.next_fr())
    mv = draw.fr_vec(pr.log2ceil(map_D))
    mu = draw.fr_vec(pr.log2ceil(map_D))
    o_map = omap.prove_pairs([int(x) % R for x in MIN], [int(x) % R for x in MOUT], mv, mu)
    assert ref_map_r == bn254.fr_to_bytes(omap.r) and ref_map_val == bn254.fr_to_bytes(o_map["claim"])

    # ---- this library, same stream
    gens_j = wl.make_generators(gctx, n_gens, seed=99)
    assert gens_j.tobytes() == ref_gens
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    d_int = gctx.upload(tensor)
    com = gctx.alloc(rows * 96)
    g.commit_i32(gctx, table, d_int, size, wd, com)
    assert g.decode_jacobian(gctx.download(com, rows * 96).reshape(-1, 24)) == ref_c0
    d_fr = gctx.alloc(size * 32)
    gctx.fr_from_i32(d_int, size, d_fr)
    g.commit_fr(gctx, table, d_fr, size, wd, com)
    assert g.decode_jacobian(gctx.download(com, rows * 96).reshape(-1, 24)) == ref_c1
    e2 = host.decode_field(gctx.random_fr(pr.log2ceil(size)))
    c2 = host.decode_field(gctx.random_fr(1))[0]
    assert e2 == e and c2 == c
    mine = host.hyrax_open(gctx, table, d_fr, size, N, layer_num, e2, c2, gens_j[0])
    assert mine.result_raw.tobytes() == ref_result and mine.z_raw.tobytes() == ref_z
    assert mine["com_d"] == ref_com_d and mine["com_ad"] == ref_com_ad
    u2 = host.decode_field(gctx.random_fr(len(u)))
    v2 = host.decode_field(gctx.random_fr(len(v)))
    ma, mb, mf, _ = host.prove_matmul(gctx, gctx.fr_upload([int(x) for x in A]), gctx.fr_upload([int(x) for x in B]),
                                      L, Nn, M, K, u2, v2, claim)
    assert tuple(bn254.fr_to_bytes(x) for x in (ma, mb, mf)) == (ref_a, ref_b, ref_final)
    lkm = host.Lookup(gctx, -(lk_len // 2), lk_len)
    lv2 = host.decode_field(gctx.random_fr(len(lv)))
    dS = gctx.fr_upload([int(x) for x in Q])
    value, _ = lkm.prove(dS, lk_D, gctx.alloc(lk_D * 32), lv2, table=table, msm_size=n_gens // 16)
    assert bn254.fr_to_bytes(value) == ref_lookup
    lkm.close()
    eu2, ev2 = host.decode_field(gctx.random_fr(6)), host.decode_field(gctx.random_fr(6))
    m_ea, m_eb, _, _ = host.prove_elemul(gctx, gctx.fr_upload(fa), gctx.fr_upload(fb), eL, eM, eN, eu2, ev2, ecl)
    assert (bn254.fr_to_bytes(m_ea), bn254.fr_to_bytes(m_eb)) == (ref_ea, ref_eb)
    us2 = [host.decode_field(gctx.random_fr(6)) for _ in range(2)]
    cv2 = host.decode_field(gctx.random_fr(6))
    m_comb, _ = host.combine_claims(gctx, gctx.fr_upload(fa), esize, [k1, k2], us2, cv2)
    assert bn254.fr_to_bytes(m_comb) == ref_comb
    mmap = host.Lookup(gctx, map_low, map_len, map_table)
    assert bn254.fr_to_bytes(mmap.r) == ref_map_r
    mv2 = host.decode_field(gctx.random_fr(len(mv)))
    m_val, _ = mmap.prove_pairs(gctx.fr_upload([int(x) for x in MIN]), gctx.fr_upload([int(x) for x in MOUT]), map_D,
                                gctx.alloc(map_D * 32), gctx.alloc(map_D * 32), mv2, table=table, msm_size=n_gens // 16)
    assert bn254.fr_to_bytes(m_val) == ref_map_val
    mmap.close()
    table.close()
