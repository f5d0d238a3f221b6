"""Golden vectors produced by the REFERENCE's own code, and the oracle check against them.

``python tests/golden/reference_vectors.py <harness> <out_dir>`` (needs a GPU and
``oracle/_ref/ref_harness``, i.e. the reference's unmodified src/*.cu built by ``make -C oracle ref``)
writes

    reference_parity_in.bin         the input blob handed to ``ref_harness parity``
    reference_parity_in.bin.table   the mapping table file the reference's tLookupRangeMapping loads
    reference_parity_out.bin        everything the reference returned

The committed copies of those three files were made that way on a B200.  ``check_oracle`` replays the
same seeded random stream through the Python oracle and compares every value; it needs no GPU, so the
oracle stays pinned to the reference wherever the tests run.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from oracle import bn254  # noqa: E402
from oracle import protocols as pr  # noqa: E402

R = bn254.R
IN_NAME, OUT_NAME = "reference_parity_in.bin", "reference_parity_out.bin"
SEED = 99                     # seed of the random stream inside ref_harness parity


def build_inputs() -> dict:
    """Shapes respect what the reference's unguarded kernels can take (row counts that fill whole
    blocks, power-of-two sizes)."""
    p = dict(n_gens=1024, N=4, layer_num=2, L=1, Nn=4, M=8, K=6, lk_len=4096, lk_D=16384, eL=2, eM=4, eN=8,
             map_len=4096, map_D=16384, map_low=-2048)
    p["size"] = 64 * p["N"] * 16
    rng = np.random.default_rng(23)
    p["tensor"] = rng.integers(-2**31, 2**31, size=p["size"], dtype=np.int64).astype(np.int32)
    p["A"] = rng.integers(-2**12, 2**12, size=p["L"] * p["Nn"] * p["K"]).astype(np.int32)
    p["B"] = rng.integers(-2**12, 2**12, size=p["L"] * p["M"] * p["K"]).astype(np.int32)
    p["Y"] = (p["A"].reshape(p["L"], p["Nn"], p["K"]).astype(np.int64)
              @ p["B"].reshape(p["L"], p["M"], p["K"]).astype(np.int64).transpose(0, 2, 1)).astype(np.int32)
    p["Q"] = rng.integers(-(p["lk_len"] // 2), p["lk_len"] // 2, size=p["lk_D"]).astype(np.int32)
    esize = p["eL"] * p["eM"] * p["eN"]
    p["EA"] = rng.integers(-2**20, 2**20, size=esize).astype(np.int32)
    p["EB"] = rng.integers(-2**20, 2**20, size=esize).astype(np.int32)
    p["map_table"] = rng.integers(-2**16, 2**16, size=p["map_len"]).astype(np.int32)
    p["MIN"] = rng.integers(p["map_low"], p["map_low"] + p["map_len"], size=p["map_D"]).astype(np.int32)
    p["MOUT"] = p["map_table"][p["MIN"] - p["map_low"]]
    return p


def write_blob(p: dict, path: Path) -> None:
    p["map_table"].tofile(str(path) + ".table")
    with open(path, "wb") as f:
        f.write(np.array([p["n_gens"], p["size"], p["N"], p["layer_num"], p["L"], p["Nn"], p["M"], p["K"], p["lk_len"],
                          p["lk_D"]], dtype=np.uint32).tobytes())
        for k in ("tensor", "A", "B", "Y", "Q"):
            f.write(p[k].tobytes())
        f.write(np.array([p["eL"], p["eM"], p["eN"], p["map_len"], p["map_D"], p["map_low"] & 0xFFFFFFFF],
                         dtype=np.uint32).tobytes())
        for k in ("EA", "EB", "MIN", "MOUT"):
            f.write(p[k].tobytes())


def read_blob(path: Path) -> dict:
    raw = Path(path).read_bytes()
    h = np.frombuffer(raw[:40], dtype=np.uint32)
    p = dict(zip(("n_gens", "size", "N", "layer_num", "L", "Nn", "M", "K", "lk_len", "lk_D"), (int(x) for x in h)))
    pos = 40

    def ints(n):
        nonlocal pos
        a = np.frombuffer(raw[pos:pos + 4 * n], dtype=np.int32).copy()
        pos += 4 * n
        return a

    p["tensor"] = ints(p["size"])
    p["A"], p["B"] = ints(p["L"] * p["Nn"] * p["K"]), ints(p["L"] * p["M"] * p["K"])
    p["Y"], p["Q"] = ints(p["L"] * p["Nn"] * p["M"]), ints(p["lk_D"])
    h2 = np.frombuffer(raw[pos:pos + 24], dtype=np.uint32)
    pos += 24
    p.update(eL=int(h2[0]), eM=int(h2[1]), eN=int(h2[2]), map_len=int(h2[3]), map_D=int(h2[4]),
             map_low=int(np.int32(h2[5])))
    esize = p["eL"] * p["eM"] * p["eN"]
    p["EA"], p["EB"] = ints(esize), ints(esize)
    p["MIN"], p["MOUT"] = ints(p["map_D"]), ints(p["map_D"])
    assert pos == len(raw)
    p["map_table"] = np.fromfile(str(path) + ".table", dtype=np.int32)
    return p


def run_reference(harness: Path, blob: Path, out: Path) -> bytes:
    env = dict(os.environ, OMP_NUM_THREADS="1")   # the reference draws the blinding vector in an OpenMP loop
    res = subprocess.run([str(harness), "parity", str(blob), str(out)], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return Path(out).read_bytes()


def parse_outputs(p: dict, raw: bytes) -> dict:
    pos = 0

    def take(n):
        nonlocal pos
        b = raw[pos:pos + n]
        pos += n
        return b

    wd = p["N"] * 16
    rows = p["size"] // wd
    o = {"wd": wd, "rows": rows}
    o["gens"] = take(p["n_gens"] * 96)
    o["c0"] = bn254.jacobian_vec_from_bytes(take(rows * 96))
    o["c1"] = bn254.jacobian_vec_from_bytes(take(rows * 96))
    o["result"], o["z"] = take(32), take(wd * 32)
    o["com_d"], o["com_ad"] = bn254.jacobian_from_bytes(take(96)), bn254.jacobian_from_bytes(take(96))
    for k in ("claim0", "a", "b", "final", "lookup", "ecl0", "ea", "eb", "k1", "k2", "comb", "map_r", "map_val"):
        o[k] = take(32)
    assert pos == len(raw)
    return o


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def check_oracle(p: dict, o: dict) -> dict:
    """Replays the reference's random stream through the oracle and asserts that every value the
    reference returned is reproduced.  Returns intermediate values the GPU test reuses."""
    fb = bn254.fr_to_bytes
    draw = bn254.SplitMix64(SEED)
    gens = [bn254.scalar_mul(draw.next_fr(), bn254.G1_GEN) for _ in range(p["n_gens"])]
    assert o["gens"] == b"".join(bn254.jacobian_to_bytes(q) for q in gens)
    wd, size, N = o["wd"], p["size"], p["N"]
    t_int = [int(x) for x in p["tensor"]]
    want_com = pr.commit_rows(t_int, wd, gens)
    assert o["c0"] == want_com and o["c1"] == want_com
    e = draw.fr_vec(pr.log2ceil(size))
    c = draw.next_fr()
    d = draw.fr_vec(wd)
    proof = pr.hyrax_open([x % R for x in t_int], e, c, size, N, p["layer_num"], gens, gens[0], d)
    assert o["result"] == fb(proof["result"]) and o["z"] == bn254.fr_vec_to_bytes(proof["z"])
    assert o["com_d"] == proof["com_d"] and o["com_ad"] == proof["com_ad"]
    L, Nn, M, K = p["L"], p["Nn"], p["M"], p["K"]
    u = draw.fr_vec(pr.log2ceil(L * Nn * M))
    v = draw.fr_vec(pr.log2ceil(K * L))
    claim = _mle([int(x) % R for x in p["Y"].reshape(-1)], u)
    a_cl, b_cl, final, _ = pr.prove_matmul([int(x) % R for x in p["A"]], [int(x) % R for x in p["B"]], L, Nn, M, K, u, v, claim)
    assert (o["claim0"], o["a"], o["b"], o["final"]) == tuple(fb(x) for x in (claim, a_cl, b_cl, final))
    lk = pr.LookupRange(-(p["lk_len"] // 2), p["lk_len"], draw.next_fr())
    lv = draw.fr_vec(pr.log2ceil(p["lk_D"]))
    lu = draw.fr_vec(pr.log2ceil(p["lk_D"]))
    got = lk.prove([int(x) % R for x in p["Q"]], lv, lu)
    assert o["lookup"] == fb(got["claim"])
    fa, fbv = [int(x) % R for x in p["EA"]], [int(x) % R for x in p["EB"]]
    esize = len(fa)
    ne = pr.log2ceil(esize)
    eu, ev = draw.fr_vec(ne), draw.fr_vec(ne)
    ecl = _mle([x * y % R for x, y in zip(fa, fbv)], eu)
    o_ea, o_eb, _, _ = pr.prove_elemul(fa, fbv, p["eL"], p["eM"], p["eN"], eu, ev, ecl)
    assert (o["ecl0"], o["ea"], o["eb"]) == tuple(fb(x) for x in (ecl, o_ea, o_eb))
    u1, u2, cv = draw.fr_vec(ne), draw.fr_vec(ne), draw.fr_vec(ne)
    k1, k2 = _mle(fa, u1), _mle(fa, u2)
    o_comb, _ = pr.combine_claims(fa, [k1, k2], [u1, u2], cv, esize)
    assert (o["k1"], o["k2"], o["comb"]) == tuple(fb(x) for x in (k1, k2, o_comb))
    omap = pr.LookupRangeMapping(p["map_low"], p["map_len"], [int(x) for x in p["map_table"]], draw.next_fr(), draw.next_fr())
    mv = draw.fr_vec(pr.log2ceil(p["map_D"]))
    mu = draw.fr_vec(pr.log2ceil(p["map_D"]))
    o_map = omap.prove_pairs([int(x) % R for x in p["MIN"]], [int(x) % R for x in p["MOUT"]], mv, mu)
    assert o["map_r"] == fb(omap.r) and o["map_val"] == fb(o_map["claim"])
    return {"gens": gens, "e": e, "c": c, "u": u, "v": v, "claim": claim, "lv": lv, "fa": fa, "fb": fbv, "ecl": ecl,
            "k1": k1, "k2": k2, "mv": mv}


if __name__ == "__main__":
    harness, out_dir = Path(sys.argv[1]), Path(sys.argv[2])
    out_dir.mkdir(parents=True, exist_ok=True)
    params = build_inputs()
    write_blob(params, out_dir / IN_NAME)
    raw_out = run_reference(harness, out_dir / IN_NAME, out_dir / OUT_NAME)
    check_oracle(params, parse_outputs(params, raw_out))
    print("reference vectors written to", out_dir, "and reproduced by the oracle")
