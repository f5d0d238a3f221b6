"""The C++ veneer (include/grape_veneer.hpp) reproduces the reference's host API: a driver written
like the reference's test/*.cu programs is compiled with g++, run on the GPU, and every value it
produces is compared with the oracle."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import bn254, cport
from oracle import protocols as pr

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
R = bn254.R


def _mle(t, u):
    n = 1 << len(u)
    return pr.partial_eval(list(t) + [0] * (n - len(t)), n, u, n, 0, 1)[0]


def test_cpp_driver_matches_oracle(tmp_path):
    exe = tmp_path / "veneer_driver"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(ROOT / "tests/cpp/veneer_driver.cpp"),
                    "-L", str(ROOT / "grape_b200"), "-lgrape_b200", f"-Wl,-rpath,{ROOT / 'grape_b200'}", "-o", str(exe)],
                   check=True)
    n_gens, N, layer_num = 512, 4, 2
    size = layer_num * 2 * N * 16
    L, Nn, M, K = 1, 4, 8, 6
    lk_len, lk_D = 1024, 4096
    rng = np.random.default_rng(17)
    gens = bn254.make_generators(n_gens, seed=3)
    gj = np.frombuffer(b"".join(bn254.jacobian_to_bytes(g) for g in gens), dtype=np.uint32).reshape(-1, 24)
    table = cport.table_build(gj)  # the reference's points.bin layout
    tensor = rng.integers(-2**31, 2**31, size=size, dtype=np.int64).astype(np.int32)
    A = rng.integers(-2**12, 2**12, size=L * Nn * K).astype(np.int32)
    B = rng.integers(-2**12, 2**12, size=L * M * K).astype(np.int32)
    Y = (A.reshape(L, Nn, K).astype(np.int64) @ B.reshape(L, M, K).astype(np.int64).transpose(0, 2, 1)).astype(np.int32)
    Q = rng.integers(-(lk_len // 2), lk_len // 2, size=lk_D).astype(np.int32)
    blob = tmp_path / "in.bin"
    with open(blob, "wb") as f:
        f.write(np.array([n_gens, size, N, layer_num, L, Nn, M, K, lk_len, lk_D], dtype=np.uint32).tobytes())
        f.write(table.tobytes())
        f.write(gj[0].tobytes())
        for arr in (tensor, A, B, Y, Q):
            f.write(arr.tobytes())
    out = tmp_path / "out.bin"
    res = subprocess.run([str(exe), str(blob), str(out)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    raw = out.read_bytes()
    pos = 0

    def take(n):
        nonlocal pos
        b = raw[pos:pos + n]
        pos += n
        return b

    # oracle, with the same random stream (seed 99) consumed in the driver's order
    draw = bn254.SplitMix64(99)
    wd = N * 16
    rows = size // wd
    t_int = [int(x) for x in tensor]
    want_com = b"".join(bn254.jacobian_to_bytes(p) for p in pr.commit_rows(t_int, wd, gens))
    assert take(rows * 96) == want_com                      # Hyrax::commit(int*)
    assert take(rows * 96) == want_com                      # Hyrax::commit(FrTensor&)
    e = draw.fr_vec(pr.log2ceil(size))
    c = draw.next_fr()
    d = draw.fr_vec(wd)
    proof = pr.hyrax_open([x % R for x in t_int], e, c, size, N, layer_num, gens, gens[0], d)
    assert take(32) == bn254.fr_to_bytes(proof["result"])
    assert take(wd * 32) == bn254.fr_vec_to_bytes(proof["z"])
    assert take(96) == bn254.jacobian_to_bytes(proof["com_d"])
    assert take(96) == bn254.jacobian_to_bytes(proof["com_ad"])
    u = draw.fr_vec(pr.log2ceil(L * Nn * M))
    v = draw.fr_vec(pr.log2ceil(K * L))
    claim = _mle([int(x) % R for x in Y.reshape(-1)], u)
    a_cl, b_cl, final, _ = pr.prove_matmul([int(x) % R for x in A], [int(x) % R for x in B], L, Nn, M, K, u, v, claim)
    assert take(32) == bn254.fr_to_bytes(claim)
    assert take(32) == bn254.fr_to_bytes(a_cl)
    assert take(32) == bn254.fr_to_bytes(b_cl)
    assert take(32) == bn254.fr_to_bytes(final)
    assert np.frombuffer(take(4), dtype=np.uint32)[0] == 1  # the wrong claim threw std::runtime_error
    lk = pr.LookupRange(-(lk_len // 2), lk_len, draw.next_fr())
    lv = draw.fr_vec(pr.log2ceil(lk_D))
    lu = draw.fr_vec(pr.log2ceil(lk_D))
    got = lk.prove([int(x) % R for x in Q], lv, lu)
    assert take(32) == bn254.fr_to_bytes(got["claim"])
    assert take(32) == bn254.fr_to_bytes((a_cl * (1 << 16) + got["claim"]) % R)
    assert pos == len(raw)
