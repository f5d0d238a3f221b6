"""Proof of the feed-forward half of one (batch of) LLaMA-2 decoder layer(s): the call sequence of
the reference's end-to-end driver, test/llm.cu:73-262, on top of this package's provers.

Tensors are the quantised intermediates the reference's data producer dumps (zzllama/llama/model.py):
for every matmul Y = X W^T the quotient q = round(Y / s) and remainder rem = Y - q s are stored and
the prover (i) range-checks rem with a lookup, (ii) opens it, (iii) continues with the claim
q~(e) s + rem~(e) (test/llm.cu:98-108).  `synthesize_ffn` produces self-consistent tensors of any
shape from a seed; the reference reads them from files that are not distributable.

The walk is backwards from the block output, exactly in the reference's order:
  open(output) -> down_out (value, remainder lookup) -> matmul down (+ open W_down)
  -> upSilu remainder -> Hadamard up_out * silu_out -> SwiGLU mapping lookup on (gate_out, silu_out)
  -> up_out remainder -> matmul up (+ open W_up) -> gate_out remainder (scale 2) -> matmul gate
  (+ open W_gate) -> combine the two claims on the block input.
Every junction the reference asserts is checked here and raises `ProofError`.
"""
from __future__ import annotations

import contextlib
import time
from dataclasses import dataclass, field

import numpy as np

from . import host
from .host import Context, GeneratorTable, Lookup, decode_field, reassemble_vectors

R = host.FR_MODULUS


class ProofError(RuntimeError):
    pass


def log2ceil(n: int) -> int:
    return max(n - 1, 0).bit_length()


@dataclass
class FFNShape:
    layer_num: int
    tokens: int
    dim: int
    ffn: int
    scale1: int = 1 << 16          # matmul rescale (reference SCALE1)
    scale2: int = 1 << 20          # SwiGLU gate rescale (reference SCALE2)
    swiglu_low: int = -(1 << 18)   # mapping table range (reference: tLookupRangeMapping(-(1<<18), 1<<19, ...))
    swiglu_len: int = 1 << 19
    npoints: int = 16384           # reference global `npoints`: msm_size of the wide lookups

    @property
    def ffn_pad(self) -> int:
        return 1 << log2ceil(self.ffn)


def round_div(x: np.ndarray, s: int):
    q = np.floor_divide(x + s // 2, s)
    return q, x - q * s


def synthesize_ffn(shape: FFNShape, seed: int, x_range: int = 1 << 13, w_std: float = 0.02 * 65536,
                   matmul=None, x=None, skip=None):
    """Self-consistent integer tensors of the FFN block.  `matmul(a, b)` multiplies int64 arrays
    [..., n, k] x [..., m, k]^T exactly (default: numpy int64).  `x` (block input) and `skip`
    (residual added to the block output) are drawn at random unless given."""
    rng = np.random.default_rng(seed)
    L, T, d, F = shape.layer_num, shape.tokens, shape.dim, shape.ffn
    if matmul is None:
        matmul = lambda a, b: np.einsum("lnk,lmk->lnm", a, b)
    if x is None:
        x = rng.integers(-x_range, x_range, size=(L, T, d)).astype(np.int64)
    x = np.asarray(x, dtype=np.int64)
    wgen = lambda *s: np.clip(np.rint(rng.normal(0, w_std, size=s)), -(1 << 15), (1 << 15) - 1).astype(np.int64)
    W_up, W_gate, W_down = wgen(L, F, d), wgen(L, F, d), wgen(L, d, F)
    table = np.clip(np.rint(rng.normal(0, shape.scale1, size=shape.swiglu_len)), -(1 << 30), (1 << 30)).astype(np.int64)
    table[-shape.swiglu_low] = 0  # f(0) = 0, as for SiLU: zero padding of the ffn axis stays inside the relation
    up_q, up_rem = round_div(matmul(x, W_up), shape.scale1)
    gate_q, gate_rem = round_div(matmul(x, W_gate), shape.scale2)
    if gate_q.min() < shape.swiglu_low or gate_q.max() >= shape.swiglu_low + shape.swiglu_len:
        raise ValueError("gate values leave the SwiGLU table; lower x_range / w_std")
    silu = table[gate_q - shape.swiglu_low]
    upsilu_q, upsilu_rem = round_div(up_q * silu, shape.scale1)
    down_q, down_rem = round_div(matmul(upsilu_q, W_down), shape.scale1)
    if skip is None:
        skip = rng.integers(-x_range, x_range, size=(L, T, d)).astype(np.int64)
    skip = np.asarray(skip, dtype=np.int64)
    t = {"x": x, "W_up": W_up, "W_gate": W_gate, "W_down": W_down, "up_q": up_q, "up_rem": up_rem, "gate_q": gate_q,
         "gate_rem": gate_rem, "silu": silu, "upsilu_q": upsilu_q, "upsilu_rem": upsilu_rem, "down_q": down_q,
         "down_rem": down_rem, "output": down_q + skip, "swiglu_table": table}
    for k, v in t.items():
        if np.abs(v).max() >= 1 << 31:
            raise ValueError(f"{k} does not fit int32")
    return {k: v.astype(np.int32) for k, v in t.items()}


@dataclass
class FFNTrace:
    """Values at the junctions of the walk (what a verifier would receive besides the openings)."""
    values: dict = field(default_factory=dict)
    opens: int = 0
    lookups: int = 0
    matmuls: int = 0
    seconds: dict = field(default_factory=dict)  # wall time per kind of step (filled when timing is on)
    steps: list = field(default_factory=list)    # (kind, seconds) of every step in walk order (timing on)


class FFNProver:
    """Holds the lookup tables and the generator table; `prove` walks one block."""

    def __init__(self, ctx: Context, shape: FFNShape, table: GeneratorTable, G_jacobian: np.ndarray,
                 swiglu_table: np.ndarray):
        self.ctx, self.shape, self.table, self.G = ctx, shape, table, G_jacobian
        s = shape
        # draw order of the reference: the opening scalar c first (test/llm.cu:52), then the lookup
        # objects' alpha / r in construction order (test/llm.cu:54-64)
        self.c = decode_field(ctx.random_fr(1))[0]
        self.rs = Lookup(ctx, -(s.scale1 // 2), s.scale1)
        self.swiglu_rs = Lookup(ctx, -(s.scale2 // 2), s.scale2)
        self.swiglu = Lookup(ctx, s.swiglu_low, s.swiglu_len, swiglu_table)

    timing = False  # set to True to synchronise around every step and fill FFNTrace.seconds
    prefetch_inputs = False  # set to True (page-locked inputs) to upload all tensors behind the first steps

    @contextlib.contextmanager
    def _phase(self, trace, name):
        if not self.timing:
            yield
            return
        self.ctx.sync()
        t0 = time.perf_counter()
        yield
        self.ctx.sync()
        dt = time.perf_counter() - t0
        trace.seconds[name] = trace.seconds.get(name, 0.0) + dt
        trace.steps.append((name, dt))

    # -- helpers ---------------------------------------------------------------------------------
    # Device buffers are recycled between steps (the reference keeps three preallocated tensors for
    # the same reason: allocating and freeing multi-gigabyte buffers per step costs more than the proof).
    def _alloc(self, nbytes: int):
        pool = self.__dict__.setdefault("_pool", [])
        best = None
        for b in pool:
            if nbytes <= b.nbytes <= 2 * max(nbytes, 1) and (best is None or b.nbytes < best.nbytes):
                best = b
        if best is not None:
            pool.remove(best)
            return best
        return self.ctx.alloc(nbytes)

    def _release(self, *bufs):
        self.__dict__.setdefault("_pool", []).extend(bufs)

    def _clone(self, src, nbytes: int):
        buf = self._alloc(nbytes)
        self.ctx._check(self.ctx.lib.grape_d2d(self.ctx.handle, buf.ptr, src.ptr, nbytes))
        return buf

    def release_pool(self):
        for b in self.__dict__.pop("_pool", []):
            b.free()

    def prefetch(self, t: dict):
        """Starts the upload of every large int32 tensor of `t` on the copy stream (they should be
        page-locked), so that the copies run behind the first proof steps; `_fr` picks them up."""
        import ctypes as C
        staged = self.__dict__.setdefault("_staged", {})
        # copies are issued in the order the previous walk consumed the tensors (the copy stream is a
        # queue: a tensor needed first must not wait behind the others); first walk: dictionary order
        seen = self.__dict__.get("_use_order", [])
        rank = {key: i for i, key in enumerate(seen)}
        big = [v for v in t.values() if isinstance(v, np.ndarray) and v.dtype == np.int32 and v.nbytes >= (1 << 20)
               and v.flags.c_contiguous]
        big.sort(key=lambda v: rank.get(v.ctypes.data, len(rank)))
        self._use_order = []
        for v in big:
            key = v.ctypes.data
            if key in staged:
                continue
            buf = self._alloc(v.nbytes)
            tk = C.c_uint32()
            self.ctx._check(self.ctx.lib.grape_h2d_prefetch(self.ctx.handle, buf.ptr, key, v.nbytes, C.byref(tk)))
            staged[key] = (buf, tk.value, v)     # keeps the host array alive until the copy is consumed

    def _fr(self, ints: np.ndarray):
        """int32 host tensor -> Fr tensor on the device, sized for row padding of the ffn axis."""
        flat = np.ascontiguousarray(ints, dtype=np.int32).reshape(-1)
        t0 = time.perf_counter()
        self.__dict__.setdefault("_use_order", []).append(flat.ctypes.data)
        hit = self.__dict__.get("_staged", {}).pop(flat.ctypes.data, None)
        if hit is not None:
            d_int = hit[0]
            self.ctx._check(self.ctx.lib.grape_prefetch_wait(self.ctx.handle, hit[1]))
        else:
            d_int = self._alloc(flat.nbytes)
            self.ctx._check(self.ctx.lib.grape_h2d(self.ctx.handle, d_int.ptr, flat.ctypes.data, flat.nbytes))
        if self.timing:   # from page-locked host arrays the copy is asynchronous; wait only to attribute time
            self.ctx.sync()
            self.upload_seconds = getattr(self, "upload_seconds", 0.0) + time.perf_counter() - t0
        cap = flat.size
        if flat.size % self.shape.ffn == 0 and self.shape.ffn != self.shape.ffn_pad:
            cap = flat.size // self.shape.ffn * self.shape.ffn_pad
        buf = self._alloc(cap * 32)
        self.ctx.fr_from_i32(d_int, flat.size, buf)
        self._release(d_int)
        return buf, flat.size

    def _draw(self, n: int):
        return decode_field(self.ctx.random_fr(n))

    def _open(self, buf, size: int, e, N: int, trace: FFNTrace):
        trace.opens += 1
        # the z vectors of a walk land in page-locked buffers that belong to the prover and are
        # reused by the next walk (one per opening, in order): the proof's output area
        zbufs = self.__dict__.setdefault("_zbufs", [])
        new_n = (1 << log2ceil(N)) * 16
        k = trace.opens - 1
        if k == len(zbufs) or (k < len(zbufs) and zbufs[k].shape[0] != new_n):
            arr = self.ctx.pinned_array((new_n, 8), np.uint32)
            if k == len(zbufs):
                zbufs.append(arr)
            else:
                zbufs[k] = arr
        with self._phase(trace, "open"):
            return host.hyrax_open(self.ctx, self.table, buf, size, N, self.shape.layer_num, e, self.c, self.G,
                                   z_out=zbufs[k])

    def _rescale(self, lk: Lookup, rem_ints, e, msm: int, open_N: int, q_claim: int, scale: int, trace, name):
        """Remainder lookup + opening + claim algebra (test/llm.cu:98-108 pattern)."""
        s = self.shape
        rem, size = self._fr(rem_ints)
        keep = self._clone(rem, size * 32)
        cap = (1 << log2ceil(size))
        A = self._alloc(cap * 32)
        trace.lookups += 1
        with self._phase(trace, "lookup"):
            lookup_value, _ = lk.prove(rem, size, A, e, inner=s.ffn, inner_pad=s.ffn_pad, table=self.table, msm_size=msm)
        proof = self._open(keep, size, e, open_N, trace)
        if proof["result"] != lookup_value:
            raise ProofError(f"{name}: opening of the remainder disagrees with the lookup claim")
        self._release(rem, keep, A)
        value = (q_claim * scale + lookup_value) % R
        trace.values[name] = value
        return value

    # -- the walk ----------------------------------------------------------------------------------
    def prove(self, t: dict) -> FFNTrace:
        ctx, s = self.ctx, self.shape
        L, T, d, F = s.layer_num, s.tokens, s.dim, s.ffn
        lT, ld, lF = log2ceil(T), log2ceil(d), log2ceil(F)
        trace = FFNTrace()
        if self.prefetch_inputs:
            self.prefetch(t)
        # output opening and the skip split (test/llm.cu:75-92)
        out, size = self._fr(t["output"])
        e1 = self._draw(log2ceil(size))
        proof = self._open(out, size, e1, size // L // T, trace)
        self._release(out)
        dq, _ = self._fr(t["down_q"])
        down_out_value = ctx.fr_eval(dq, size, e1)
        self._release(dq)
        trace.values["skip"] = (proof["result"] - down_out_value) % R
        skip_eval_point = list(e1)
        down_out_value = self._rescale(self.rs, t["down_rem"], e1, d, size // L // T, down_out_value, s.scale1, trace, "down_out")
        # matmul down (test/llm.cu:111-125)
        A, _ = self._fr(t["upsilu_q"])
        W, wsize = self._fr(t["W_down"])
        Wkeep = self._clone(W, wsize * 32)
        e2 = self._draw(log2ceil(F * L))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            a_cl, b_cl, _, _ = host.prove_matmul(ctx, A, W, L, T, d, F, e1, e2, down_out_value)
        e1, e2 = reassemble_vectors(e1, e2, lT, lF, ld)
        proof = self._open(Wkeep, wsize, e2, F, trace)
        if proof["result"] != b_cl:
            raise ProofError("down: opening of W_down disagrees with the sumcheck claim")
        self._release(A, W, Wkeep)
        # upSilu remainder (test/llm.cu:128-138)
        upsilu_value = self._rescale(self.rs, t["upsilu_rem"], e1, s.npoints, F, a_cl, s.scale1, trace, "upSilu")
        # Hadamard product up_out * silu_out (test/llm.cu:140-150)
        up, esize = self._fr(t["up_q"])
        silu, _ = self._fr(t["silu"])
        silu_keep = self._clone(silu, esize * 32)
        e2 = self._draw(log2ceil(esize))
        with self._phase(trace, "elemul"):
            up_cl, silu_cl, _, _ = host.prove_elemul(ctx, up, silu, L, T, F, e1, e2, upsilu_value)
        trace.values["silu_at_e2"] = silu_cl
        self._release(up, silu)
        # SwiGLU mapping lookup on (gate_out, silu_out) (test/llm.cu:153-166)
        gate, gsize = self._fr(t["gate_q"])
        e1 = self._draw(log2ceil(gsize))
        cap = 1 << log2ceil(gsize)
        work, Abuf = self._alloc(cap * 32), self._alloc(cap * 32)
        trace.lookups += 1
        with self._phase(trace, "lookup"):
            lookup_value, _ = self.swiglu.prove_pairs(gate, silu_keep, gsize, work, Abuf, e1, inner=F, inner_pad=s.ffn_pad,
                                                      table=self.table, msm_size=s.npoints)
        gate_out_value = self._open(gate, gsize, e1, F, trace)["result"]
        silu_open = self._open(silu_keep, gsize, e1, F, trace)["result"]
        if lookup_value != (gate_out_value + silu_open * self.swiglu.r) % R:
            raise ProofError("swiglu: lookup claim disagrees with the two openings")
        self._release(gate, silu_keep, work, Abuf)
        # up_out remainder (test/llm.cu:169-178)
        up_out_value = self._rescale(self.rs, t["up_rem"], e2, s.npoints, F, up_cl, s.scale1, trace, "up_out")
        # matmul up (test/llm.cu:181-198)
        x, xsize = self._fr(t["x"])
        x_keep = self._clone(x, xsize * 32)
        W, wsize = self._fr(t["W_up"])
        Wkeep = self._clone(W, wsize * 32)
        e3 = self._draw(log2ceil(d * L))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            n1, w_cl, _, _ = host.prove_matmul(ctx, x, W, L, T, F, d, e2, e3, up_out_value)
        e2, e3 = reassemble_vectors(e2, e3, lT, ld, lF)
        if self._open(Wkeep, wsize, e3, d, trace)["result"] != w_cl:
            raise ProofError("up: opening of W_up disagrees with the sumcheck claim")
        self._release(x, W, Wkeep)
        # gate_out remainder at the second scale (test/llm.cu:204-213)
        gate_out_value = self._rescale(self.swiglu_rs, t["gate_rem"], e1, s.npoints, F, gate_out_value, s.scale2, trace, "gate_out")
        # matmul gate (test/llm.cu:216-231)
        x2 = self._clone(x_keep, xsize * 32)
        W, wsize = self._fr(t["W_gate"])
        Wkeep = self._clone(W, wsize * 32)
        e3 = self._draw(log2ceil(d * L))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            n2, w_cl, _, _ = host.prove_matmul(ctx, x2, W, L, T, F, d, e1, e3, gate_out_value)
        e1, e3 = reassemble_vectors(e1, e3, lT, ld, lF)
        if self._open(Wkeep, wsize, e3, d, trace)["result"] != w_cl:
            raise ProofError("gate: opening of W_gate disagrees with the sumcheck claim")
        self._release(x2, W, Wkeep)
        # both claims on the block input become one (test/llm.cu:234-239)
        e3 = self._draw(log2ceil(d * L * T))
        with self._phase(trace, "combine"):
            value, _ = host.combine_claims(ctx, x_keep, d * L * T, [n1, n2], [e2, e1], e3)
        self._release(x_keep)
        trace.values["normOutSecond"] = value
        trace.values["normOutSecond_point"] = e3
        trace.values["skip_point"] = skip_eval_point
        return trace
