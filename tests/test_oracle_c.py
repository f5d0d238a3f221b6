"""Pins the C restatement (oracle/grape_oracle.c) to the big-integer oracle (oracle/bn254.py)."""
import random

import numpy as np

from oracle import bn254, cport
from oracle import protocols as pr

R, P = bn254.R, bn254.P


def _enc(vals, mod):
    return np.frombuffer(b"".join(bn254.fe_to_bytes(v, mod) for v in vals), dtype=np.uint32).reshape(-1, 8)


def _dec(arr, mod):
    raw = np.ascontiguousarray(arr).tobytes()
    return [bn254.fe_from_bytes(raw[i:i + 32], mod) for i in range(0, len(raw), 32)]


def test_field_ops_match_bigint():
    rng = random.Random(1)
    for name, mod in (("fr", R), ("fp", P)):
        a = [0, 1, mod - 1, mod - 2] + [rng.randrange(mod) for _ in range(300)]
        b = [mod - 1, mod - 1, mod - 1, 5] + [rng.randrange(mod) for _ in range(300)]
        A, B = _enc(a, mod), _enc(b, mod)
        assert _dec(cport.fe_binary(name, "add", A, B), mod) == [(x + y) % mod for x, y in zip(a, b)]
        assert _dec(cport.fe_binary(name, "sub", A, B), mod) == [(x - y) % mod for x, y in zip(a, b)]
        assert _dec(cport.fe_binary(name, "mul", A, B), mod) == [x * y % mod for x, y in zip(a, b)]


def test_from_i32():
    x = np.array([0, 1, -1, 2**31 - 1, -2**31, 65536, -40000], dtype=np.int32)
    assert cport.fr_from_i32(x).tobytes() == bn254.fr_vec_to_bytes([int(v) for v in x])


def test_table_and_commits_match_bigint():
    gens = bn254.make_generators(16, seed=9)
    gj = np.frombuffer(b"".join(bn254.jacobian_to_bytes(g) for g in gens), dtype=np.uint32).reshape(-1, 24)
    table = cport.table_build(gj)
    assert bn254.affine_from_bytes(table[0, 3].tobytes()) is None
    assert bn254.affine_from_bytes(table[1, 3].tobytes()) == gens[3]
    assert bn254.affine_from_bytes(table[255, 7].tobytes()) == bn254.scalar_mul(255, gens[7])
    rng = random.Random(2)
    s = [rng.randrange(-2**31, 2**31) for _ in range(16 * 5)]
    s[:4] = [0, -2**31, 2**31 - 1, -1]
    got = cport.commit_i32(np.array(s, dtype=np.int32), 16, table)
    want = pr.commit_rows(s, 16, gens)
    assert got.tobytes() == b"".join(bn254.jacobian_to_bytes(p) for p in want)
    # a row range only
    part = cport.commit_i32(np.array(s, dtype=np.int32), 16, table, 2, 4)
    assert part.tobytes() == got[2:4].tobytes()
    f = [rng.randrange(R) for _ in range(32)]
    got = cport.commit_fr(_enc(f, R), 16, table)
    want = pr.commit_rows(f, 16, gens)
    assert got.tobytes() == b"".join(bn254.jacobian_to_bytes(p) for p in want)


def test_fold_matches_bigint():
    rng = random.Random(4)
    for other, c, gap in [(2, 6, 3), (1, 11, 1), (3, 8, 4), (1, 1, 5)]:
        n = other * c * gap
        t = [rng.randrange(R) for _ in range(n)]
        x = [rng.randrange(R) for _ in range(6)]
        got = _dec(cport.fr_fold(_enc(t, R), n, _enc(x, R), c, 1, gap), R)
        assert got == pr.partial_eval(t, n, x, c, 1, gap)


def test_c_prove_matmul_matches_python_oracle():
    """The C restatement of prove_matmul (one layer) against the Python one: claims, every round
    polynomial, and the failing-round report on a wrong claim."""
    import random
    from oracle import protocols as pr
    R = bn254.R
    rnd = random.Random(8)
    for N, M, K in ((4, 8, 6), (3, 2, 11), (2, 2, 64)):
        A = [rnd.randrange(-2**15, 2**15) for _ in range(N * K)]
        B = [rnd.randrange(-2**15, 2**15) for _ in range(M * K)]
        u = [rnd.randrange(R) for _ in range(pr.log2ceil(N * M) + 1)]
        v = [rnd.randrange(R) for _ in range(pr.log2ceil(K))]
        a_ = pr.partial_eval([x % R for x in A], N * K, u, N, pr.log2ceil(M), K)
        b_ = pr.partial_eval([x % R for x in B], M * K, u, M, 0, K)
        claim = sum(x * y for x, y in zip(a_, b_)) % R
        want = pr.prove_matmul([x % R for x in A], [x % R for x in B], 1, N, M, K, u, v, claim)
        enc = lambda xs: np.frombuffer(bn254.fr_vec_to_bytes(xs), dtype=np.uint32).reshape(-1, 8)
        rc, a, b, final, tr = cport.prove_matmul_l1(np.array(A, dtype=np.int32), np.array(B, dtype=np.int32), N, M, K,
                                                    enc(u), enc(v), enc([claim]))
        assert rc == 0
        assert bn254.fr_from_bytes(a.tobytes()) == want[0] and bn254.fr_from_bytes(b.tobytes()) == want[1]
        assert bn254.fr_from_bytes(final.tobytes()) == want[2]
        got_tr = [bn254.fr_vec_from_bytes(tr[i].tobytes()) for i in range(tr.shape[0])]
        assert got_tr == [list(p) for p in want[3]]
        rc_bad = cport.prove_matmul_l1(np.array(A, dtype=np.int32), np.array(B, dtype=np.int32), N, M, K, enc(u), enc(v),
                                       enc([(claim + 1) % R]))[0]
        assert rc_bad == 1   # the first round's check fails, where the reference throws


def test_c_lookup_range_matches_python_oracle():
    """The C restatement of tLookupRange::prove against the Python one: multiplicities, S~(v), the
    final claim and every round polynomial; a query outside the table is reported."""
    import random
    from oracle import protocols as pr
    R = bn254.R
    rnd = random.Random(12)
    enc = lambda xs: np.frombuffer(bn254.fr_vec_to_bytes(xs), dtype=np.uint32).reshape(-1, 8)
    for low, N, D in ((-8, 16, 64), (0, 4, 4), (-128, 256, 1024)):
        q = [rnd.randrange(low, low + N) for _ in range(D)]
        alpha = rnd.randrange(R)
        lD = pr.log2ceil(D)
        u = [rnd.randrange(R) for _ in range(lD)]
        v = [rnd.randrange(R) for _ in range(lD)]
        want = pr.LookupRange(low, N, alpha).prove([x % R for x in q], v, u)
        rc, m, s_claim, final, tr = cport.lookup_range(np.array(q, dtype=np.int32), low, N, enc([alpha])[0], enc(u), enc(v))
        assert rc == 0
        assert [int(x) for x in m] == want["m"]
        assert bn254.fr_from_bytes(s_claim.tobytes()) == want["claim"]
        assert bn254.fr_from_bytes(final.tobytes()) == want["final"]
        got = [bn254.fr_vec_from_bytes(tr[i].tobytes()) for i in range(tr.shape[0])]
        assert got == [list(p) + [0] * (4 - len(p)) for p in want["transcript"]]
    q = np.array([0, 1, 2, 99], dtype=np.int32)
    assert cport.lookup_range(q, 0, 4, enc([5])[0], enc([1, 2]), enc([3, 4]))[0] == -3
