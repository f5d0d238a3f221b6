"""ctypes binding of ``libgrape_b200.so`` (the C ABI declared in ``include/grape_b200.h``).

The library is the product: if it is missing or cannot be loaded this module raises, there is no
Python or CPU stand-in for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
#: the shared library; GRAPE_B200_LIBRARY names another build of it (e.g. one compiled with other flags)
LIB_PATH = Path(os.environ.get("GRAPE_B200_LIBRARY") or PKG / "libgrape_b200.so")
HEADER = PKG.parent / "include" / "grape_b200.h"

GRAPE_OK = 0
ERR_NAMES = {1: "GRAPE_ERR_INVALID", 2: "GRAPE_ERR_CUDA", 3: "GRAPE_ERR_CHECK", 4: "GRAPE_ERR_NOMEM",
             5: "GRAPE_ERR_LIMIT"}


class GrapeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


def declared_symbols() -> list[str]:
    """Names of every function the public header declares."""
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grape_[a-z0-9_]+)\s*\(", text)))


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python grape_b200/csrc/build.py` (needs nvcc). "
            "grape_b200 has no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    _declare(lib)
    _lib = lib
    return lib


def _declare(lib):
    vp, u64, u32, i32p = C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p
    sz = C.c_size_t

    def f(name, args, res=C.c_int):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res

    f("grape_version", [])
    f("grape_ctx_create", [C.c_int, C.POINTER(vp)])
    f("grape_ctx_destroy", [vp])
    f("grape_ctx_error", [vp], C.c_char_p)
    f("grape_ctx_sync", [vp])
    f("grape_ctx_stream", [vp], vp)
    f("grape_ctx_launches", [vp], u64)
    f("grape_ctx_status", [vp, C.POINTER(u32)])
    f("grape_rng_seed", [vp, u64])
    f("grape_rng_fr", [vp, vp, u64])
    f("grape_dev_alloc", [vp, sz, C.POINTER(vp)])
    f("grape_dev_free", [vp, vp])
    f("grape_h2d", [vp, vp, vp, sz])
    f("grape_h2d_prefetch", [vp, vp, vp, sz, C.POINTER(u32)])
    f("grape_prefetch_wait", [vp, u32])
    f("grape_d2h", [vp, vp, vp, sz])
    f("grape_d2d", [vp, vp, vp, sz])
    f("grape_dev_zero", [vp, vp, sz])
    f("grape_host_alloc_pinned", [vp, sz, C.POINTER(vp)])
    f("grape_host_free_pinned", [vp, vp])
    f("grape_table_create", [vp, vp, u32, u32, u32, C.POINTER(vp)])
    f("grape_bls12_381_table_create", [vp, vp, u32, u32, u32, C.POINTER(vp)])
    f("grape_table_curve", [vp], u32)
    f("grape_bls12_381_field_binary", [vp, C.c_int, C.c_int, vp, vp, vp, u64])
    f("grape_bls12_381_fr_from_i32", [vp, vp, vp, u64])
    f("grape_bls12_381_measure_mul_peak", [vp, C.POINTER(C.c_double)])
    f("grape_table_from_reference", [vp, vp, u32, C.POINTER(vp)])
    f("grape_table_destroy", [vp])
    f("grape_table_bytes", [vp], u64)
    f("grape_table_data", [vp], vp)
    f("grape_commit_i32", [vp, vp, i32p, u64, u32, u32, vp])
    f("grape_commit_fr", [vp, vp, vp, u64, u32, vp])
    f("grape_commit_i32_host", [vp, vp, vp, u64, u32, u32, vp])
    f("grape_fr_from_i32", [vp, vp, vp, u64])
    f("grape_fr_from_u32", [vp, vp, vp, u64])
    f("grape_fr_to_mont", [vp, vp, u64])
    f("grape_fr_from_mont", [vp, vp, u64])
    for name in ("grape_fr_add", "grape_fr_sub", "grape_fr_mul", "grape_fr_scale", "grape_fr_add_scalar"):
        f(name, [vp, vp, vp, vp, u64])
    f("grape_fp_binary", [vp, C.c_int, vp, vp, vp, u64])
    f("grape_fr_axpy", [vp, vp, vp, vp, vp, u64])
    f("grape_fr_inverse", [vp, vp, vp, vp, u64])
    f("grape_pad_i32", [vp, vp, vp, u32, u32, u64])
    f("grape_fr_pad", [vp, vp, vp, u32, u32, u64, vp])
    f("grape_fr_sum", [vp, vp, u64, vp])
    f("grape_fr_rowsum", [vp, vp, vp, u64, u32])
    f("grape_fr_fold", [vp, vp, u64, vp, u32, u64, vp])
    f("grape_fold_i32", [vp, vp, u64, vp, u32, u64, vp])
    f("grape_measure_int_peak", [vp, C.c_int, C.POINTER(C.c_double)])
    f("grape_measure_madd_peak", [vp, C.POINTER(C.c_double)])
    f("grape_diag_field_check", [vp, C.c_int, vp, u64, C.POINTER(u32)])
    f("grape_timer_begin", [vp])
    f("grape_timer_end", [vp, C.POINTER(C.c_float)])
    f("grape_prof_enable", [vp, C.c_int])
    f("grape_prof_read", [vp, C.POINTER(C.c_float), C.POINTER(u32)])
    f("grape_prove_matmul", [vp, vp, vp, u32, u32, u32, u32, vp, u32, vp, u32, vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_lookup_set_bucket_commit", [vp, C.c_int])
    f("grape_prove_matmul_i32", [vp, vp, vp, u32, u32, u32, u32, vp, u32, vp, u32, vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_prove_matmul_partial", [vp, vp, vp, u32, u32, u32, u32, vp, u32, vp, u32, vp, C.POINTER(u32)])
    f("grape_prove_matmul_finish", [vp, vp, u32, u32, u32, u32, u32, vp, u32, vp, u32, vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_prove_elemul", [vp, vp, vp, u32, u32, u32, vp, u32, vp, u32, vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_combine_claims", [vp, vp, u64, vp, u32, vp, vp, u32, vp, vp, u32, C.POINTER(u32)])
    f("grape_lookup_range_create", [vp, C.c_int32, u32, C.POINTER(vp)])
    f("grape_lookup_mapping_create", [vp, C.c_int32, u32, vp, C.POINTER(vp)])
    f("grape_lookup_destroy", [vp])
    f("grape_lookup_params", [vp, vp, vp, vp, C.POINTER(u32)])
    f("grape_lookup_table", [vp, C.c_int], vp)
    f("grape_lookup_last_proof", [vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_lookup_prove_range", [vp, vp, vp, u64, vp, vp, u32, u32, u32, vp, u32, vp, vp, vp, vp, u32, C.POINTER(u32)])
    f("grape_lookup_prove_mapping", [vp, vp, vp, vp, u64, vp, vp, vp, u32, u32, u32, vp, u32, vp, vp, vp, vp, u32,
                                     C.POINTER(u32)])
    f("grape_hyrax_open", [vp, vp, vp, u64, u32, u32, vp, u32, vp, vp, vp, vp, vp, vp])
    f("grape_g1_lincomb", [vp, vp, vp, u64, vp])
    for name in ("grape_hg1_add", "grape_hg1_scalar_mul"):
        f(name, [vp, vp, vp], None)
    for name in ("grape_hg1_neg", "grape_hg1_normalise"):
        f(name, [vp, vp], None)
    f("grape_hg1_equal", [vp, vp])
    for name in _OPTIONAL:
        if hasattr(lib, name):
            f(name, _OPTIONAL[name])


# entry points added by later parts of the library register their signatures here
_OPTIONAL: dict[str, list] = {
    "grape_commit_set_affine": [C.c_void_p, C.c_int, C.c_int, C.c_int],
    "grape_host_device_pointer": [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)],
    "grape_commit_i32_static": [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint32,
                                C.c_uint32, C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)],
}
