"""ctypes loader for ``oracle/liboracle.so`` (the C restatement in ``grape_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for full-size parity cases and the host-core baseline the
benchmark reports.  ``build()`` compiles it with gcc.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"


def build(force: bool = False) -> Path:
    src = HERE / "grape_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        # -march=native is avoided: the library is built here and run on another machine
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-std=c11", "-shared", "-o", str(LIB), str(src)],
                       check=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = C.CDLL(str(LIB))
        vp, u64, u32 = C.c_void_p, C.c_uint64, C.c_uint32
        _lib.oracle_threads.restype = C.c_int
        _lib.oracle_fe_binary.argtypes = [C.c_int, C.c_int, vp, vp, vp, u64]
        _lib.oracle_fr_from_i32.argtypes = [vp, vp, u64]
        _lib.oracle_table_build.argtypes = [vp, u64, vp]
        _lib.oracle_commit_i32.argtypes = [vp, u64, u64, u64, vp, u64, vp]
        _lib.oracle_commit_fr.argtypes = [vp, u64, u64, u64, vp, u64, vp]
        _lib.oracle_fr_fold.argtypes = [vp, u64, vp, u32, u32, u64]
    return _lib


def threads() -> int:
    return lib().oracle_threads()


def fe_binary(field: str, op: str, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint32).reshape(-1, 8)
    b = np.ascontiguousarray(b, dtype=np.uint32).reshape(-1, 8)
    out = np.empty_like(a)
    lib().oracle_fe_binary({"fr": 0, "fp": 1}[field], {"add": 0, "sub": 1, "mul": 2}[op],
                           a.ctypes.data, b.ctypes.data, out.ctypes.data, a.shape[0])
    return out


def fr_from_i32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.int32).reshape(-1)
    out = np.empty((x.size, 8), dtype=np.uint32)
    lib().oracle_fr_from_i32(x.ctypes.data, out.ctypes.data, x.size)
    return out


def table_build(gens_jacobian: np.ndarray) -> np.ndarray:
    """uint32[n, 24] generators -> uint32[256, n, 16] table, row w = w * G_i (reference layout)."""
    g = np.ascontiguousarray(gens_jacobian, dtype=np.uint32).reshape(-1, 24)
    n = g.shape[0]
    table = np.empty((256, n, 16), dtype=np.uint32)
    lib().oracle_table_build(g.ctypes.data, n, table.ctypes.data)
    return table


def commit_i32(scalars: np.ndarray, wd: int, table: np.ndarray, row_begin: int = 0, row_end: int | None = None):
    s = np.ascontiguousarray(scalars, dtype=np.int32).reshape(-1)
    rows = s.size // wd
    row_end = rows if row_end is None else row_end
    out = np.empty((row_end - row_begin, 24), dtype=np.uint32)
    lib().oracle_commit_i32(s.ctypes.data, wd, row_begin, row_end, table.ctypes.data, table.shape[1],
                            out.ctypes.data)
    return out


def commit_fr(scalars: np.ndarray, wd: int, table: np.ndarray, row_begin: int = 0, row_end: int | None = None):
    s = np.ascontiguousarray(scalars, dtype=np.uint32).reshape(-1, 8)
    rows = s.shape[0] // wd
    row_end = rows if row_end is None else row_end
    out = np.empty((row_end - row_begin, 24), dtype=np.uint32)
    lib().oracle_commit_fr(s.ctypes.data, wd, row_begin, row_end, table.ctypes.data, table.shape[1],
                           out.ctypes.data)
    return out


def fr_fold(t: np.ndarray, ntot: int, x: np.ndarray, c: int, idx: int, gap: int) -> np.ndarray:
    """The reference's in-place fold; returns the compacted [other][gap] front of the buffer."""
    t = np.array(t, dtype=np.uint32).reshape(-1, 8).copy()
    x = np.ascontiguousarray(x, dtype=np.uint32).reshape(-1, 8)
    lib().oracle_fr_fold(t.ctypes.data, ntot, x.ctypes.data, c, idx, gap)
    return t[: ntot // c]


def prove_matmul_l1(A: np.ndarray, B: np.ndarray, N: int, M: int, K: int, u: np.ndarray, v: np.ndarray, claim: np.ndarray):
    """``prove_matmul`` for one layer on int32 tensors A [N][K], B [M][K]; u, v, claim are uint32[*, 8]
    Montgomery records.  Returns (rc, a_claim, b_claim, final_claim, transcript[rounds, 3, 8])."""
    A = np.ascontiguousarray(A, dtype=np.int32).reshape(-1)
    B = np.ascontiguousarray(B, dtype=np.int32).reshape(-1)
    u = np.ascontiguousarray(u, dtype=np.uint32).reshape(-1, 8)
    v = np.ascontiguousarray(v, dtype=np.uint32).reshape(-1, 8)
    cl = np.array(claim, dtype=np.uint32).reshape(8).copy()
    rounds = max(K - 1, 0).bit_length()
    a, b = np.zeros(8, dtype=np.uint32), np.zeros(8, dtype=np.uint32)
    tr = np.zeros((max(rounds, 1), 3, 8), dtype=np.uint32)
    f = lib().oracle_prove_matmul_l1
    f.restype = C.c_int
    rc = f(C.c_void_p(A.ctypes.data), C.c_void_p(B.ctypes.data), C.c_uint32(N), C.c_uint32(M), C.c_uint32(K),
           C.c_void_p(u.ctypes.data), C.c_void_p(v.ctypes.data), C.c_void_p(cl.ctypes.data), C.c_void_p(a.ctypes.data),
           C.c_void_p(b.ctypes.data), C.c_void_p(tr.ctypes.data))
    return rc, a, b, cl, tr[:rounds]


def lookup_range(q: np.ndarray, low: int, n_table: int, alpha: np.ndarray, u: np.ndarray, v: np.ndarray):
    """``tLookupRange::prove`` on a power-of-two number of int32 queries.  alpha, u, v: uint32[*, 8]
    Montgomery records.  Returns (rc, multiplicities uint32[n_table], S~(v), final claim, transcript[rounds, 4, 8])."""
    q = np.ascontiguousarray(q, dtype=np.int32).reshape(-1)
    lD, lN = (q.size - 1).bit_length(), (n_table - 1).bit_length()
    assert q.size == 1 << lD and n_table == 1 << lN and lN <= lD
    alpha = np.ascontiguousarray(alpha, dtype=np.uint32).reshape(8)
    u = np.ascontiguousarray(u, dtype=np.uint32).reshape(-1, 8)
    v = np.ascontiguousarray(v, dtype=np.uint32).reshape(-1, 8)
    assert u.shape[0] == lD and v.shape[0] == lD
    m = np.zeros(n_table, dtype=np.uint32)
    s_claim, final = np.zeros(8, dtype=np.uint32), np.zeros(8, dtype=np.uint32)
    tr = np.zeros((max(lD, 1), 4, 8), dtype=np.uint32)
    f = lib().oracle_lookup_range
    f.restype = C.c_int
    rc = f(C.c_void_p(q.ctypes.data), C.c_uint32(lD), C.c_int32(low), C.c_uint32(lN), C.c_void_p(alpha.ctypes.data),
           C.c_void_p(u.ctypes.data), C.c_void_p(v.ctypes.data), C.c_void_p(m.ctypes.data), C.c_void_p(s_claim.ctypes.data),
           C.c_void_p(final.ctypes.data), C.c_void_p(tr.ctypes.data))
    return rc, m, s_claim, final, tr[:lD]


if __name__ == "__main__":
    print(build(force=True))
