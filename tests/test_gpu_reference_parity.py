"""Pins this library (and the oracle) against the reference's own code.

``oracle/_ref/ref_harness`` is the reference's unmodified src/*.cu linked with a libff stand-in
(oracle/ref_shim) and built by ``make -C oracle ref`` where the reference tree is available.  The
harness runs the reference's commit (int and Fr), open, prove_matmul, prove_eleMul, combine_claims,
tLookupRange::prove and tLookupRangeMapping::prove on a blob of inputs with a seeded random stream.
When the harness is present it is run here and must reproduce the committed golden output byte for
byte; either way the same inputs and the same stream then go through the oracle and through
libgrape_b200, and every value is compared.  Shapes respect what the reference's unguarded kernels
can take (row counts that fill whole blocks, power-of-two sizes).
"""
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import bn254
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
HARNESS = ROOT / "oracle" / "_ref" / "ref_harness"
GOLDEN = ROOT / "tests" / "golden"
sys.path.insert(0, str(GOLDEN))
R = bn254.R


def test_reference_outputs_equal_oracle_and_library(gctx, tmp_path):
    import grape_b200 as g
    import reference_vectors as rv
    from grape_b200 import host, workloads as wl
    p = rv.build_inputs()
    raw = (GOLDEN / rv.OUT_NAME).read_bytes()
    if HARNESS.exists():   # the reference itself, run now on this GPU
        rv.write_blob(p, tmp_path / rv.IN_NAME)
        live = rv.run_reference(HARNESS, tmp_path / rv.IN_NAME, tmp_path / rv.OUT_NAME)
        assert live == raw
    o = rv.parse_outputs(p, raw)
    vals = rv.check_oracle(p, o)
    n_gens, N, layer_num, size = p["n_gens"], p["N"], p["layer_num"], p["size"]
    L, Nn, M, K = p["L"], p["Nn"], p["M"], p["K"]
    lk_len, lk_D, eL, eM, eN = p["lk_len"], p["lk_D"], p["eL"], p["eM"], p["eN"]
    map_len, map_D, map_low, map_table = p["map_len"], p["map_D"], p["map_low"], p["map_table"]
    tensor, A, B, Q, MIN, MOUT = p["tensor"], p["A"], p["B"], p["Q"], p["MIN"], p["MOUT"]
    esize = eL * eM * eN
    wd, rows = o["wd"], o["rows"]
    ref_gens, ref_c0, ref_c1, ref_result, ref_z = o["gens"], o["c0"], o["c1"], o["result"], o["z"]
    ref_com_d, ref_com_ad = o["com_d"], o["com_ad"]
    ref_a, ref_b, ref_final, ref_lookup = o["a"], o["b"], o["final"], o["lookup"]
    ref_ea, ref_eb, ref_comb, ref_map_r, ref_map_val = o["ea"], o["eb"], o["comb"], o["map_r"], o["map_val"]
    e, c, u, v, claim, lv = vals["e"], vals["c"], vals["u"], vals["v"], vals["claim"], vals["lv"]
    fa, fb, ecl, k1, k2, mv = vals["fa"], vals["fb"], vals["ecl"], vals["k1"], vals["k2"], vals["mv"]

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
