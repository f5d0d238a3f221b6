"""Python host side over the C ABI: contexts, device buffers, generator tables and the
field-tensor / commitment calls, with numpy arrays as the host representation.

Field elements travel as ``uint32[n, 8]`` arrays (little-endian limbs of the Montgomery residue),
affine points as ``uint32[n, 16]``, Jacobian points as ``uint32[n, 24]`` -- the byte layouts of the
reference's ``fr_t`` / ``affine_t`` / ``jacob_t``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import GrapeError

FR_MODULUS = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001
FP_MODULUS = 0x30644E72E131A029B85045B68181585D97816A916871CA8D3C208C16D87CFD47
_MONT = 1 << 256
COM_SCALE = 16


# ----------------------------------------------------------------------------- encoding helpers
def encode_field(values, modulus=FR_MODULUS) -> np.ndarray:
    """Python integers (any sign) -> uint32[n, 8] Montgomery limbs."""
    out = np.empty((len(values), 8), dtype=np.uint32)
    buf = bytearray()
    for v in values:
        buf += ((int(v) % modulus) * _MONT % modulus).to_bytes(32, "little")
    out[:] = np.frombuffer(bytes(buf), dtype="<u4").reshape(-1, 8)
    return out


def decode_field(arr: np.ndarray, modulus=FR_MODULUS) -> list[int]:
    """uint32[n, 8] Montgomery limbs -> Python integers in [0, modulus)."""
    arr = np.ascontiguousarray(arr, dtype="<u4").reshape(-1, 8)
    rinv = pow(_MONT, -1, modulus)
    raw = arr.tobytes()
    return [int.from_bytes(raw[i:i + 32], "little") * rinv % modulus for i in range(0, len(raw), 32)]


def encode_jacobian(points) -> np.ndarray:
    """Affine (x, y) tuples or None (infinity) -> uint32[n, 24] Jacobian records with Z = 1."""
    vals = []
    for p in points:
        vals += [1, 1, 0] if p is None else [p[0], p[1], 1]
    return encode_field(vals, FP_MODULUS).reshape(-1, 24)


def decode_jacobian(arr: np.ndarray):
    """uint32[n, 24] Jacobian records -> affine (x, y) tuples, None for infinity."""
    flat = decode_field(np.ascontiguousarray(arr).reshape(-1, 8), FP_MODULUS)
    out = []
    for i in range(0, len(flat), 3):
        X, Y, Z = flat[i:i + 3]
        if Z == 0:
            out.append(None)
        else:
            zi = pow(Z, -1, FP_MODULUS)
            out.append((X * zi * zi % FP_MODULUS, Y * zi * zi * zi % FP_MODULUS))
    return out


# ----------------------------------------------------------------------------- context / buffers
class DeviceBuffer:
    """A cudaMalloc'd region owned by a context."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        ctx._check(ctx.lib.grape_dev_alloc(ctx.handle, self.nbytes, C.byref(p)))
        self.ptr = p.value or 0

    def free(self):
        if self.ptr and self.ctx.handle:
            self.ctx.lib.grape_dev_free(self.ctx.handle, self.ptr)
        self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def at(self, byte_offset: int) -> int:
        return self.ptr + int(byte_offset)


class Context:
    """One GPU, one stream, one scratch arena, one seedable random stream."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        rc = self.lib.grape_ctx_create(int(device), C.byref(h))
        if rc != 0:
            raise GrapeError(rc, f"cannot create a context on CUDA device {device} (no GPU?)")
        self.handle = h.value
        self.device = device

    def close(self):
        if self.handle:
            self.lib.grape_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise GrapeError(rc, self.lib.grape_ctx_error(self.handle).decode())

    # -- memory
    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def upload(self, arr: np.ndarray) -> DeviceBuffer:
        arr = np.ascontiguousarray(arr)
        buf = DeviceBuffer(self, max(arr.nbytes, 1))
        if arr.nbytes:
            self._check(self.lib.grape_h2d(self.handle, buf.ptr, arr.ctypes.data, arr.nbytes))
            self.sync()
        return buf

    def download(self, src, nbytes: int, dtype=np.uint32, offset: int = 0) -> np.ndarray:
        ptr = (src.ptr if isinstance(src, DeviceBuffer) else int(src)) + offset
        out = np.empty(nbytes // np.dtype(dtype).itemsize, dtype=dtype)
        self._check(self.lib.grape_d2h(self.handle, out.ctypes.data, ptr, nbytes))
        return out

    def clone(self, src, nbytes: int) -> DeviceBuffer:
        """Device-to-device copy into a fresh buffer."""
        buf = DeviceBuffer(self, max(nbytes, 1))
        if nbytes:
            self._check(self.lib.grape_d2d(self.handle, buf.ptr, _p(src), nbytes))
        return buf

    def sync(self):
        self._check(self.lib.grape_ctx_sync(self.handle))

    def status(self) -> int:
        f = C.c_uint32()
        self._check(self.lib.grape_ctx_status(self.handle, C.byref(f)))
        return f.value

    @property
    def launches(self) -> int:
        return int(self.lib.grape_ctx_launches(self.handle))

    @property
    def stream(self) -> int:
        return int(self.lib.grape_ctx_stream(self.handle) or 0)

    def timer_begin(self):
        self._check(self.lib.grape_timer_begin(self.handle))

    def timer_end(self) -> float:
        """Milliseconds on the context's stream since ``timer_begin`` (synchronises)."""
        ms = C.c_float()
        self._check(self.lib.grape_timer_end(self.handle, C.byref(ms)))
        return ms.value

    def prof_enable(self, on: bool = True):
        self._check(self.lib.grape_prof_enable(self.handle, int(on)))

    def prof_read(self):
        """(total milliseconds, launches) of the dominant kernels recorded since the last read."""
        ms, n = C.c_float(), C.c_uint32()
        self._check(self.lib.grape_prof_read(self.handle, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def pinned_array(self, shape, dtype) -> np.ndarray:
        """A numpy array over page-locked host memory (kept alive by the context)."""
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self._check(self.lib.grape_host_alloc_pinned(self.handle, max(nbytes, 1), C.byref(p)))
        buf = (C.c_char * nbytes).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype).reshape(shape)
        self._pinned = getattr(self, "_pinned", []) + [(p.value, buf)]
        return arr

    def host_device_pointer(self, arr: np.ndarray) -> int:
        """Device-side address of a page-locked numpy array (``pinned_array``): kernels read it in place."""
        p = C.c_void_p()
        self._check(self.lib.grape_host_device_pointer(self.handle, arr.ctypes.data, C.byref(p)))
        return p.value

    def measure_int_peak(self, kind: int) -> float:
        """Measured integer-pipe ceiling (ops/s): 0 mad.lo, 1 mad.wide, 2 lo/hi pairs, 3 field muls."""
        v = C.c_double()
        self._check(self.lib.grape_measure_int_peak(self.handle, kind, C.byref(v)))
        return v.value

    def measure_bls12_381_mul_peak(self) -> float:
        """12-limb base-field multiplications per second on register operands."""
        v = C.c_double()
        self._check(self.lib.grape_bls12_381_measure_mul_peak(self.handle, C.byref(v)))
        return v.value

    def measure_madd_peak(self) -> float:
        """Mixed point additions per second with register-resident operands."""
        v = C.c_double()
        self._check(self.lib.grape_measure_madd_peak(self.handle, C.byref(v)))
        return v.value

    def field_check(self, field: int, d_elems, n: int) -> int:
        """Failure mask of the squaring / inversion self-check over n elements of field 0 BN254 Fp,
        1 BN254 Fr, 2 BLS12-381 Fp, 3 BLS12-381 Fr (0 = every identity holds)."""
        m = C.c_uint32()
        self._check(self.lib.grape_diag_field_check(self.handle, field, _p(d_elems), n, C.byref(m)))
        return m.value

    def set_bucket_commit(self, mode: int):
        """How lookups commit A: 0 never by the bucket method, 1 when cheaper (default), 2 whenever possible."""
        self._check(self.lib.grape_lookup_set_bucket_commit(self.handle, mode))

    def set_affine_commit(self, mode: int, slots_per_lane: int = 0, chunks: int = 0):
        """Which kernel accumulates row commitments: 0 extended coordinates only, 1 affine accumulators with
        shared inversions where the cost model expects a gain, 2 always affine (slots_per_lane / chunks: 0 = chosen).
        A new context uses 1 for Fr scalars and 0 for int32 scalars; this sets both, -1 restores that."""
        self._check(self.lib.grape_commit_set_affine(self.handle, mode, slots_per_lane, chunks))

    # -- randomness seam
    def seed(self, seed: int):
        self._check(self.lib.grape_rng_seed(self.handle, seed))

    def random_fr(self, n: int) -> np.ndarray:
        out = np.empty((n, 8), dtype=np.uint32)
        self._check(self.lib.grape_rng_fr(self.handle, out.ctypes.data, n))
        return out

    # -- field tensors (device pointers in, device pointers out)
    def fr_upload(self, values) -> DeviceBuffer:
        return self.upload(encode_field(values))

    def fr_download(self, buf, n: int, offset_elems: int = 0) -> list[int]:
        return decode_field(self.download(buf, n * 32, offset=offset_elems * 32))

    def fr_from_i32(self, d_in, n, d_out):
        self._check(self.lib.grape_fr_from_i32(self.handle, _p(d_in), _p(d_out), n))

    def fr_from_u32(self, d_in, n, d_out):
        self._check(self.lib.grape_fr_from_u32(self.handle, _p(d_in), _p(d_out), n))

    def fr_binary(self, op: str, a, b, out, n):
        fn = {"add": self.lib.grape_fr_add, "sub": self.lib.grape_fr_sub, "mul": self.lib.grape_fr_mul,
              "scale": self.lib.grape_fr_scale, "add_scalar": self.lib.grape_fr_add_scalar}[op]
        self._check(fn(self.handle, _p(a), _p(b), _p(out), n))

    def fp_binary(self, op: str, a, b, out, n):
        self._check(self.lib.grape_fp_binary(self.handle, {"add": 0, "sub": 1, "mul": 2}[op], _p(a), _p(b), _p(out), n))

    def fr_to_mont(self, t, n):
        self._check(self.lib.grape_fr_to_mont(self.handle, _p(t), n))

    def fr_from_mont(self, t, n):
        self._check(self.lib.grape_fr_from_mont(self.handle, _p(t), n))

    def fr_inverse(self, d_in, d_out, n, d_shift=None):
        self._check(self.lib.grape_fr_inverse(self.handle, _p(d_in), _p(d_shift), _p(d_out), n))

    def fr_sum(self, d_in, n, d_out):
        self._check(self.lib.grape_fr_sum(self.handle, _p(d_in), n, _p(d_out)))

    def fr_rowsum(self, d_in, d_out, rows, dim):
        self._check(self.lib.grape_fr_rowsum(self.handle, _p(d_in), _p(d_out), rows, dim))

    def fr_fold(self, d_t, ntot, d_x, c, gap, d_out):
        self._check(self.lib.grape_fr_fold(self.handle, _p(d_t), ntot, _p(d_x), c, gap, _p(d_out)))

    def fr_eval(self, d_t, size: int, u, inner: int | None = None) -> int:
        """Multilinear evaluation of a tensor at u (``FrTensor::operator()(vector<Fr>)``); the tensor is
        left intact.  ``inner``: row length when the size is not a power of two (rows are padded to a
        power of two with zeros; the reference hard-codes 11008)."""
        du = self.fr_upload(u)
        out = self.alloc(32)
        if size == 1 << len(u):
            self.fr_fold(d_t, size, du, size, 1, out)
        else:
            assert inner and size % inner == 0
            lin = max(inner - 1, 0).bit_length()
            tmp = self.alloc(inner * 32)
            self.fr_fold(d_t, size, du.at(lin * 32), size // inner, inner, tmp)
            self.fr_fold(tmp, inner, du, inner, 1, out)
        return self.fr_download(out, 1)[0]

    def fold_i32(self, d_t, ntot, d_x, c, gap, d_out):
        self._check(self.lib.grape_fold_i32(self.handle, _p(d_t), ntot, _p(d_x), c, gap, _p(d_out)))

    def fr_pad(self, d_in, d_out, n, pad_n, pad_size, d_pad_value):
        self._check(self.lib.grape_fr_pad(self.handle, _p(d_in), _p(d_out), n, pad_n, pad_size, _p(d_pad_value)))

    def pad_i32(self, d_in, d_out, n, pad_n, pad_size):
        self._check(self.lib.grape_pad_i32(self.handle, _p(d_in), _p(d_out), n, pad_n, pad_size))


def _p(x):
    if x is None:
        return None
    if isinstance(x, DeviceBuffer):
        return x.ptr
    return int(x)


# ----------------------------------------------------------------------------- commitments
class GeneratorTable:
    """Fixed-base table of the Hyrax generators (replaces ``precompute_generators``)."""

    def __init__(self, ctx: Context, gens_jacobian: np.ndarray, window_bits: int = 8, n_windows: int = 1,
                 curve: str = "bn254"):
        """``curve`` is "bn254" (96-byte Jacobian generator records) or "bls12_381" (144-byte)."""
        if curve not in ("bn254", "bls12_381"):
            raise ValueError("curve must be 'bn254' or 'bls12_381'")
        self.ctx = ctx
        self.curve = curve
        #: bytes of one commitment (Jacobian) record on this curve
        self.jacobian_bytes = 96 if curve == "bn254" else 144
        gens = np.ascontiguousarray(gens_jacobian, dtype=np.uint32).reshape(-1, self.jacobian_bytes // 4)
        self.n_gens = gens.shape[0]
        self.window_bits = window_bits
        self.n_windows = n_windows
        self._gens_dev = ctx.upload(gens)
        h = C.c_void_p()
        create = ctx.lib.grape_table_create if curve == "bn254" else ctx.lib.grape_bls12_381_table_create
        ctx._check(create(ctx.handle, self._gens_dev.ptr, self.n_gens, window_bits, n_windows, C.byref(h)))
        self.handle = h.value

    @property
    def nbytes(self) -> int:
        return int(self.ctx.lib.grape_table_bytes(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            self.ctx.sync()
            self.ctx.lib.grape_table_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def commit_i32(ctx: Context, table: GeneratorTable, d_scalars, size: int, wd: int, d_out, max_bits: int = 32):
    ctx._check(ctx.lib.grape_commit_i32(ctx.handle, table.handle, _p(d_scalars), size, wd, max_bits, _p(d_out)))


def commit_fr(ctx: Context, table: GeneratorTable, d_scalars, size: int, wd: int, d_out):
    ctx._check(ctx.lib.grape_commit_fr(ctx.handle, table.handle, _p(d_scalars), size, wd, _p(d_out)))


def commit_i32_host(ctx: Context, table: GeneratorTable, scalars: np.ndarray, wd: int, max_bits: int = 32,
                    out: np.ndarray | None = None) -> np.ndarray:
    """Host int32 tensor in, host Jacobian records (uint32[rows, 24], or [rows, 36] on BLS12-381) out;
    copies included."""
    scalars = np.ascontiguousarray(scalars, dtype=np.int32).reshape(-1)
    rows = scalars.size // wd
    if out is None:
        out = np.empty((rows, table.jacobian_bytes // 4), dtype=np.uint32)
    ctx._check(ctx.lib.grape_commit_i32_host(ctx.handle, table.handle, scalars.ctypes.data, scalars.size, wd,
                                             max_bits, out.ctypes.data))
    return out


def reassemble_vectors(first, second, first_size: int, same_size: int, last_size: int):
    """``ReassembleVectors`` (src/ec_operation.cu:74-122): the two points at which prove_matmul's
    returned claims hold; returns the new (first, second)."""
    r1 = list(second[:same_size]) + list(first[last_size:last_size + first_size]) + list(second[same_size:])
    r2 = list(second[:same_size]) + list(first[:last_size]) + list(second[same_size:])
    return r1, r2


# ----------------------------------------------------------------------------- sumcheck provers
def _fr_host(values) -> np.ndarray:
    return np.ascontiguousarray(encode_field(values))


def prove_matmul(ctx: Context, d_A, d_B, L: int, N: int, M: int, K: int, u, v, claim: int):
    """``prove_matmul``: returns (A_claim, B_claim, final_claim, transcript) as Python integers; the
    transcript is a list of 4-coefficient round polynomials (degree-2 rounds end with a zero).
    d_A and d_B are consumed."""
    hu, hv = _fr_host(u), _fr_host(v)
    hc = _fr_host([claim])
    out = np.zeros((2, 8), dtype=np.uint32)
    cap = len(u) + len(v) + 4
    tr = np.zeros((cap, 4, 8), dtype=np.uint32)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_prove_matmul(ctx.handle, _p(d_A), _p(d_B), L, N, M, K, hu.ctypes.data, len(u),
                                          hv.ctypes.data, len(v), hc.ctypes.data, out.ctypes.data,
                                          tr.ctypes.data, cap, C.byref(nr)))
    a, b = decode_field(out)
    polys = [decode_field(tr[i]) for i in range(nr.value)]
    return a, b, decode_field(hc)[0], polys


def prove_matmul_i32(ctx: Context, d_A_i32, d_B_i32, L: int, N: int, M: int, K: int, u, v, claim: int):
    """:func:`prove_matmul` on the int32 device tensors the Fr tensors would be built from (inputs kept)."""
    hu, hv = _fr_host(u), _fr_host(v)
    hc = _fr_host([claim])
    out = np.zeros((2, 8), dtype=np.uint32)
    cap = len(u) + len(v) + 4
    tr = np.zeros((cap, 4, 8), dtype=np.uint32)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_prove_matmul_i32(ctx.handle, _p(d_A_i32), _p(d_B_i32), L, N, M, K, hu.ctypes.data, len(u),
                                              hv.ctypes.data, len(v), hc.ctypes.data, out.ctypes.data,
                                              tr.ctypes.data, cap, C.byref(nr)))
    a, b = decode_field(out)
    polys = [decode_field(tr[i]) for i in range(nr.value)]
    return a, b, decode_field(hc)[0], polys


def matmul_partial_elems(L: int, K_local: int) -> int:
    """Field elements one prover contributes to the exchange of the sharded ``prove_matmul``."""
    rounds = max(L - 1, 0).bit_length() + max(K_local - 1, 0).bit_length()
    return 3 * rounds + 2


def prove_matmul_partial(ctx: Context, d_A_shard, d_B_shard, L: int, N: int, M: int, K_local: int, u, v_local, d_part):
    """Step 1 of the sharded ``prove_matmul``: the local rounds on this prover's shard (columns
    k = k' * P + rank of A and B).  Writes ``matmul_partial_elems(L, K_local)`` field elements to the
    device buffer ``d_part`` (a DeviceBuffer or a raw device address); asynchronous.  Both shards are consumed."""
    hu, hv = _fr_host(u), _fr_host(v_local)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_prove_matmul_partial(ctx.handle, _p(d_A_shard), _p(d_B_shard), L, N, M, K_local,
                                                  hu.ctypes.data, len(u), hv.ctypes.data, len(v_local), _p(d_part),
                                                  C.byref(nr)))
    return nr.value


def prove_matmul_finish(ctx: Context, d_gathered, P: int, L: int, N: int, M: int, K: int, u, v, claim: int):
    """Step 2 of the sharded ``prove_matmul`` over the P provers' gathered buffers (rank order):
    same return value as :func:`prove_matmul`."""
    hu, hv = _fr_host(u), _fr_host(v)
    hc = _fr_host([claim])
    out = np.zeros((2, 8), dtype=np.uint32)
    cap = len(u) + len(v) + 4
    tr = np.zeros((cap, 4, 8), dtype=np.uint32)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_prove_matmul_finish(ctx.handle, _p(d_gathered), P, L, N, M, K, hu.ctypes.data, len(u),
                                                 hv.ctypes.data, len(v), hc.ctypes.data, out.ctypes.data,
                                                 tr.ctypes.data, cap, C.byref(nr)))
    a, b = decode_field(out)
    polys = [decode_field(tr[i]) for i in range(nr.value)]
    return a, b, decode_field(hc)[0], polys


def prove_elemul(ctx: Context, d_A, d_B, L: int, M: int, N: int, u, v, claim: int):
    hu, hv = _fr_host(u), _fr_host(v)
    hc = _fr_host([claim])
    out = np.zeros((2, 8), dtype=np.uint32)
    cap = len(u) + 4
    tr = np.zeros((cap, 4, 8), dtype=np.uint32)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_prove_elemul(ctx.handle, _p(d_A), _p(d_B), L, M, N, hu.ctypes.data, len(u),
                                          hv.ctypes.data, len(v), hc.ctypes.data, out.ctypes.data,
                                          tr.ctypes.data, cap, C.byref(nr)))
    a, b = decode_field(out)
    return a, b, decode_field(hc)[0], [decode_field(tr[i]) for i in range(nr.value)]


def combine_claims(ctx: Context, d_X, size: int, claims, us, v):
    k, nv = len(claims), len(v)
    hcl = _fr_host(claims)
    hus = _fr_host([x for uj in us for x in uj])
    hv = _fr_host(v)
    out = np.zeros((1, 8), dtype=np.uint32)
    tr = np.zeros((nv + 1, 4, 8), dtype=np.uint32)
    nr = C.c_uint32()
    ctx._check(ctx.lib.grape_combine_claims(ctx.handle, _p(d_X), size, hcl.ctypes.data, k, hus.ctypes.data,
                                            hv.ctypes.data, nv, out.ctypes.data, tr.ctypes.data, nv + 1,
                                            C.byref(nr)))
    return decode_field(out)[0], [decode_field(tr[i]) for i in range(nr.value)]


# ----------------------------------------------------------------------------- lookup argument
class Lookup:
    """``tLookupRange`` (``mapped=None``) or ``tLookupRangeMapping`` (``mapped`` = int32 table)."""

    def __init__(self, ctx: Context, low: int, length: int, mapped: np.ndarray | None = None):
        self.ctx = ctx
        h = C.c_void_p()
        if mapped is None:
            ctx._check(ctx.lib.grape_lookup_range_create(ctx.handle, low, length, C.byref(h)))
        else:
            self._map_dev = ctx.upload(np.ascontiguousarray(mapped, dtype=np.int32))
            ctx._check(ctx.lib.grape_lookup_mapping_create(ctx.handle, low, length, self._map_dev.ptr, C.byref(h)))
        self.handle = h.value
        a, b, r = (np.zeros((1, 8), dtype=np.uint32) for _ in range(3))
        n = C.c_uint32()
        ctx.lib.grape_lookup_params(self.handle, a.ctypes.data, b.ctypes.data, r.ctypes.data, C.byref(n))
        self.alpha, self.beta, self.r = decode_field(a)[0], decode_field(b)[0], decode_field(r)[0]
        self.n = n.value
        self.low = low

    def table(self, which: str) -> list[int]:
        idx = {"T": 0, "B": 1, "m": 2, "mapped": 3}[which]
        ptr = self.ctx.lib.grape_lookup_table(self.handle, idx)
        return self.ctx.fr_download(ptr, self.n)

    def prove(self, d_S, D: int, d_A, v, inner: int = 11008, inner_pad: int = 16384, table: "GeneratorTable | None" = None,
              msm_size: int = 0, d_com_A=None, d_com_m=None):
        """``tLookupRange::prove``: returns (S_claim, transcript)."""
        hv = _fr_host(v)
        out = np.zeros((1, 8), dtype=np.uint32)
        cap = len(v) + 2
        tr = np.zeros((cap, 4, 8), dtype=np.uint32)
        nr = C.c_uint32()
        ctx = self.ctx
        ctx._check(ctx.lib.grape_lookup_prove_range(ctx.handle, self.handle, _p(d_S), D, _p(d_A), hv.ctypes.data, len(v),
                                                    inner, inner_pad, table.handle if table else None, msm_size,
                                                    _p(d_com_A), _p(d_com_m), out.ctypes.data, tr.ctypes.data, cap,
                                                    C.byref(nr)))
        return decode_field(out)[0], [decode_field(tr[i]) for i in range(nr.value)]

    def prove_pairs(self, d_S_in, d_S_out, D: int, d_S_work, d_A, v, inner: int = 11008, inner_pad: int = 16384,
                    table: "GeneratorTable | None" = None, msm_size: int = 0, d_com_A=None, d_com_m=None):
        """``tLookupRangeMapping::prove``: returns (S_claim, transcript)."""
        hv = _fr_host(v)
        out = np.zeros((1, 8), dtype=np.uint32)
        cap = len(v) + 2
        tr = np.zeros((cap, 4, 8), dtype=np.uint32)
        nr = C.c_uint32()
        ctx = self.ctx
        ctx._check(ctx.lib.grape_lookup_prove_mapping(ctx.handle, self.handle, _p(d_S_in), _p(d_S_out), D, _p(d_S_work),
                                                      _p(d_A), hv.ctypes.data, len(v), inner, inner_pad,
                                                      table.handle if table else None, msm_size, _p(d_com_A),
                                                      _p(d_com_m), out.ctypes.data, tr.ctypes.data, cap, C.byref(nr)))
        return decode_field(out)[0], [decode_field(tr[i]) for i in range(nr.value)]

    def last_proof(self):
        """(finals, u) of the last proof: finals = dict(A, S, B, T, m), the five tensors of the argument
        folded to one value each; u = the prover's own draws.  What ``verifier.verify_lookup`` takes."""
        fin = np.zeros((5, 8), dtype=np.uint32)
        n = C.c_uint32()
        self.ctx._check(self.ctx.lib.grape_lookup_last_proof(self.handle, fin.ctypes.data, None, 0, C.byref(n)))
        u = np.zeros((max(n.value, 1), 8), dtype=np.uint32)
        self.ctx._check(self.ctx.lib.grape_lookup_last_proof(self.handle, None, u.ctypes.data, n.value, C.byref(n)))
        vals = decode_field(fin)
        return dict(zip(("A", "S", "B", "T", "m"), vals)), decode_field(u[:n.value])

    def close(self):
        if getattr(self, "handle", None):
            self.ctx.lib.grape_lookup_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ----------------------------------------------------------------------------- Hyrax opening
def hyrax_open(ctx: Context, table: GeneratorTable, d_tensor, size: int, N: int, layer_num: int, eval_point, c: int,
               G_jacobian: np.ndarray, z_out: np.ndarray | None = None):
    """``Hyrax::open``: returns dict(result, z, com_d, com_ad) with points as affine tuples / None.
    ``z_out``: optional uint32[new_n, 8] array that receives z (page-locked memory makes the copy
    back an order of magnitude faster than a fresh pageable array)."""
    he, hc = _fr_host(eval_point), _fr_host([c])
    G = np.ascontiguousarray(G_jacobian, dtype=np.uint32).reshape(24)
    new_n = (1 << max(N - 1, 0).bit_length()) * COM_SCALE
    res = np.zeros((1, 8), dtype=np.uint32)
    z = np.zeros((new_n, 8), dtype=np.uint32) if z_out is None else z_out
    if z.shape != (new_n, 8) or z.dtype != np.uint32 or not z.flags.c_contiguous:
        raise ValueError("z_out must be a contiguous uint32 array of shape (new_n, 8)")
    com = np.zeros((2, 24), dtype=np.uint32)
    ctx._check(ctx.lib.grape_hyrax_open(ctx.handle, table.handle, _p(d_tensor), size, N, layer_num, he.ctypes.data,
                                        len(eval_point), hc.ctypes.data, G.ctypes.data, res.ctypes.data, z.ctypes.data,
                                        com[0].ctypes.data, com[1].ctypes.data))
    return OpenProof(res, z, com)


class OpenProof:
    """Result of ``hyrax_open`` (the reference's ``Hyrax_proof``).  Holds the raw records; the Python
    integers / affine tuples are decoded on first use (decoding a long z vector is slow)."""

    def __init__(self, res: np.ndarray, z: np.ndarray, com: np.ndarray):
        self.result_raw, self.z_raw, self.com_raw = res, z, com
        self._cache = {}

    def __getitem__(self, key: str):
        if key not in self._cache:
            if key == "result":
                self._cache[key] = decode_field(self.result_raw)[0]
            elif key == "z":
                self._cache[key] = decode_field(self.z_raw)
            elif key in ("com_d", "com_ad"):
                pts = decode_jacobian(self.com_raw)
                self._cache["com_d"], self._cache["com_ad"] = pts
            elif key == "com_bytes":
                self._cache[key] = self.com_raw.tobytes()
            else:
                raise KeyError(key)
        return self._cache[key]
