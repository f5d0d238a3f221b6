"""Proof of one whole (batch of) LLaMA-2 decoder layer(s): the rest of the reference's end-to-end
driver (test/llm.cu:242-611) after the feed-forward half of ``layer.py`` — second RMSNorm, attention
output projection, softmax x V, the softmax range relation, the exp mapping lookup, the score
matmul, the Q / K / V projections, claim batching on the normalised input, first RMSNorm, and the
final opening of the layer input.  The call order, shapes, evaluation points and junction checks
are the reference's; where the reference leaves two values unlinked (the exp input versus the
scores, the SiLU claim of the Hadamard product) this driver leaves them unlinked too.

``synthesize_layer`` builds self-consistent integer tensors (single head, no RoPE, no mask, as the
reference's modified model, zzllama/llama/model.py:166-171,518,551-552).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import host
from .host import Lookup, reassemble_vectors
from .layer import FFNProver, FFNShape, FFNTrace, ProofError, log2ceil, round_div

R = host.FR_MODULUS


@dataclass
class LayerShape(FFNShape):
    scale3: int = 1 << 22            # QK^T rescale (reference: 1 << 22, test/llm.cu:425)
    exp_low: int = -(1 << 20) + 1    # exp mapping table (reference: tLookupRangeMapping(-(1<<20)+1, 1<<20, ...))
    exp_len: int = 1 << 20
    softmax_len: int = 1 << 16       # range of the softmax rounding residual (reference: tLookupRange(0, 1<<16))


def rms_factor(x: np.ndarray, scale: int, eps: float = 1e-5) -> np.ndarray:
    """The quantised RMSNorm factor of every token, in integers: for x = scale * x_real,

        rms = round(scale / sqrt(mean(x_real^2) + eps)) = round(scale^2 * sqrt(d) / sqrt(sum(x^2) + eps * d * scale^2)),

    computed as an integer square root with 16 guard bits (the model computes it in floating point,
    zzllama/llama/model.py:204,221-226: rsqrt of the mean square plus eps, times the scale, rounded).
    x: int64 [..., d]; returns int64 [...]."""
    d = x.shape[-1]
    sq = (x.astype(np.int64) ** 2).sum(axis=-1)
    e = int(round(eps * d * scale * scale))
    guard = 16
    num = (scale ** 4 * d) << (2 * guard)
    import math
    flat = [(math.isqrt(num // (int(v) + e)) + (1 << (guard - 1))) >> guard if int(v) + e > 0 else 0 for v in sq.reshape(-1)]
    return np.array(flat, dtype=np.int64).reshape(sq.shape)


def synthesize_layer(shape: LayerShape, seed: int, x_range: int = 1 << 13, w_std: float = 0.02 * 65536,
                     matmul=None, exp_max: int = 15):
    """Integer tensors of one layer batch, all relations of the quantised forward pass holding exactly."""
    rng = np.random.default_rng(seed)
    L, T, d, F = shape.layer_num, shape.tokens, shape.dim, shape.ffn
    s1 = shape.scale1
    if matmul is None:
        matmul = lambda a, b: np.einsum("lnk,lmk->lnm", a, b)
    wgen = lambda *s: np.clip(np.rint(rng.normal(0, w_std, size=s)), -(1 << 15), (1 << 15) - 1).astype(np.int64)
    t = {}
    inp = rng.integers(-x_range, x_range, size=(L, T, d)).astype(np.int64)

    def rmsnorm(x, tag):
        # per-token factor derived from the data as the model does (zzllama/llama/model.py:204,221-239):
        # rms = round(scale / sqrt(mean((x/scale)^2) + eps)) by an integer square root, then the two rescales
        # rmsw = rms (x) w / scale and out = x * rmsw / scale; the norm weights are near one (random init)
        rms = rms_factor(x, s1).reshape(L, T, 1)
        wn = rng.integers(s1 - s1 // 8, s1 + s1 // 8 + 1, size=(L, d, 1)).astype(np.int64)
        rmsw_q, rmsw_rem = round_div(matmul(rms, wn), s1)              # [L][T][d] = rms (x) w
        out_q, out_rem = round_div(x * rmsw_q, s1)
        t.update({f"rms{tag}": rms, f"wnorm{tag}": wn, f"rmsw{tag}_q": rmsw_q, f"rmsw{tag}_rem": rmsw_rem,
                  f"norm{tag}_q": out_q, f"norm{tag}_rem": out_rem})
        return out_q

    n1 = rmsnorm(inp, "1")
    WQ, WK, WV, WO = wgen(L, d, d), wgen(L, d, d), wgen(L, d, d), wgen(L, d, d)
    xk_q, xk_rem = round_div(matmul(n1, WK), s1)
    xv_q, xv_rem = round_div(matmul(WV, n1), s1)                       # stored transposed: [L][d][T]
    # The spread of a row of scores (about nine standard deviations over 2048 keys) must stay inside the
    # exp table.  With full-size random projections it does so only for some seeds, so the query
    # projection starts at half magnitude and is halved again while a row still leaves the table.
    WQ = WQ // 2
    for _ in range(6):
        xq_q, xq_rem = round_div(matmul(n1, WQ), s1)
        sc_q, sc_rem = round_div(matmul(xq_q, xk_q), shape.scale3)     # [L][T][T]
        exp_in = sc_q - sc_q.max(axis=2, keepdims=True)
        if exp_in.min() >= shape.exp_low:
            break
        WQ = WQ // 2
    else:
        raise ValueError("scores leave the exp table; lower the magnitudes")
    exp_table = np.rint(exp_max * np.exp(-np.arange(shape.exp_len)[::-1] / max(shape.exp_len / 8, 1))).astype(np.int64)
    exp_table = np.maximum(exp_table, 0)
    exp_table[-1] = exp_max                                             # f(0): the row maximum
    exp_out = exp_table[exp_in - shape.exp_low]
    ssum = exp_out.sum(axis=2, keepdims=True)
    if 2 * ssum.max() > shape.softmax_len:
        raise ValueError("softmax row sums leave the residual range")
    soft = (exp_out * s1 + ssum // 2) // ssum
    qkv_q, qkv_rem = round_div(matmul(soft, xv_q), s1)                 # [L][T][d]
    att_q, att_rem = round_div(matmul(qkv_q, WO), s1)
    skip = att_q + inp
    n2 = rmsnorm(skip, "2")
    from .layer import synthesize_ffn  # feed-forward half on x = second norm output, residual = skip
    ffn = synthesize_ffn(shape, seed + 1, x_range=x_range, w_std=w_std, matmul=matmul, x=n2, skip=skip)
    t.update({"input": inp, "W_Q": WQ, "W_K": WK, "W_V": WV, "W_O": WO, "xq_q": xq_q, "xq_rem": xq_rem, "xk_q": xk_q,
              "xk_rem": xk_rem, "xv_q": xv_q, "xv_rem": xv_rem, "scores_q": sc_q, "scores_rem": sc_rem, "exp_in": exp_in,
              "exp_out": exp_out, "softmax": soft, "qkv_q": qkv_q, "qkv_rem": qkv_rem, "atten_q": att_q,
              "atten_rem": att_rem, "skip": skip, "exp_table": exp_table})
    for k, v in t.items():
        if np.abs(v).max() >= 1 << 31:
            raise ValueError(f"{k} does not fit int32")
    out = {k: np.ascontiguousarray(v).astype(np.int32) for k, v in t.items()}
    out.update(ffn)
    return out


class LayerProver(FFNProver):
    """Lookup tables of the whole layer; ``prove_layer`` walks FFN half, then norms and attention."""

    def __init__(self, ctx, shape: LayerShape, table, G_jacobian, swiglu_table, exp_table):
        super().__init__(ctx, shape, table, G_jacobian, swiglu_table)
        self.softmax_range = Lookup(ctx, 0, shape.softmax_len)
        self.exp = Lookup(ctx, shape.exp_low, shape.exp_len, exp_table)

    # ---- motifs --------------------------------------------------------------------------------
    def _matmul_open_w(self, A_ints, W_ints, N, M, K, u, claim, trace, name, keep_A=None):
        """prove_matmul(A, W) + ReassembleVectors + opening of W (test/llm.cu:181-198 pattern).
        Returns (A claim, new u, new v)."""
        s = self.shape
        L = s.layer_num
        A = keep_A if keep_A is not None else self._fr(A_ints)[0]
        W, wsize = self._fr(W_ints)
        Wkeep = self._clone(W, wsize * 32)
        v = self._draw(log2ceil(K * L))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            a_cl, w_cl, _, _ = host.prove_matmul(self.ctx, A, W, L, N, M, K, u, v, claim)
        u2, v2 = reassemble_vectors(u, v, log2ceil(N), log2ceil(K), log2ceil(M))
        if self._open(Wkeep, wsize, v2, K, trace)["result"] != w_cl:
            raise ProofError(f"{name}: opening of the weight disagrees with the sumcheck claim")
        self._release(A, W, Wkeep)
        return a_cl, u2, v2

    def _norm(self, t, tag, x_ints, value, e3, trace, extra_claim=None):
        """RMSNorm block walked backwards (test/llm.cu:242-310 and :540-592).
        value: claim on the norm output (quotient) at e3.  Returns (claim on x at e1, e1)."""
        ctx, s = self.ctx, self.shape
        L, T, d = s.layer_num, s.tokens, s.dim
        lT, ld = log2ceil(T), log2ceil(d)
        size = L * T * d
        value = self._rescale(self.rs, t[f"norm{tag}_rem"], e3, d, d, value, s.scale1, trace, f"norm{tag}")
        x, _ = self._fr(x_ints)
        x_keep = self._clone(x, size * 32)
        rmsw, _ = self._fr(t[f"rmsw{tag}_q"])
        e1 = self._draw(log2ceil(size))
        with self._phase(trace, "elemul"):
            x_cl, rmsw_cl, _, _ = host.prove_elemul(ctx, x, rmsw, L, T, d, e3, e1, value)
        self._release(x, rmsw)
        rmsw_value = self._rescale(self.rs, t[f"rmsw{tag}_rem"], e1, d, d, rmsw_cl, s.scale1, trace, f"rmsw{tag}")
        # rmsw = rms (x) w_norm: a matmul with inner dimension 1 (test/llm.cu:289-305)
        e3n = self._draw(log2ceil(L))
        rms, rsize = self._fr(t[f"rms{tag}"])
        wn, wsize = self._fr(t[f"wnorm{tag}"])
        rms_keep, wn_keep = self._clone(rms, rsize * 32), self._clone(wn, wsize * 32)
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            rms_cl, wn_cl, _, _ = host.prove_matmul(ctx, rms, wn, L, T, d, 1, e1, e3n, rmsw_value)
        e2, e3n = reassemble_vectors(e1, e3n, lT, 0, ld)
        if self._open(wn_keep, wsize, e3n, d // 16, trace)["result"] != wn_cl:
            raise ProofError(f"norm{tag}: opening of the norm weight disagrees")
        if self._open(rms_keep, rsize, e2, T // 16, trace)["result"] != rms_cl:
            raise ProofError(f"norm{tag}: opening of the rms factor disagrees")
        self._release(rms, wn, rms_keep, wn_keep)
        return x_cl, e1, x_keep

    # ---- the walk ----------------------------------------------------------------------------------
    def prove_layer(self, t: dict) -> FFNTrace:
        ctx, s = self.ctx, self.shape
        L, T, d = s.layer_num, s.tokens, s.dim
        lT, ld = log2ceil(T), log2ceil(d)
        size = L * T * d
        trace = self.prove(t)                                  # feed-forward half, test/llm.cu:73-239
        skip_value, skip_point = trace.values["skip"], trace.values["skip_point"]
        # ---- second norm (test/llm.cu:242-315): skip * rmsw2 -> normOutSecond
        x_cl, e1, skip_keep = self._norm(t, "2", t["skip"], trace.values["normOutSecond"],
                                         trace.values["normOutSecond_point"], trace)
        e2 = self._draw(log2ceil(size))
        with self._phase(trace, "combine"):
            skip_value, _ = host.combine_claims(ctx, skip_keep, size, [skip_value, x_cl], [skip_point, e1], e2)
        self._release(skip_keep)
        # ---- residual: skip = atten_out + input (test/llm.cu:319-326)
        inp, _ = self._fr(t["input"])
        input_value = self._open(inp, size, e2, d, trace)["result"]
        self._release(inp)
        atten_value = (skip_value - input_value) % R
        atten_value = self._rescale(self.rs, t["atten_rem"], e2, d, d, atten_value, s.scale1, trace, "atten_out")
        # ---- output projection (test/llm.cu:341-355)
        qkv_cl, e2, _ = self._matmul_open_w(t["qkv_q"], t["W_O"], T, d, d, e2, atten_value, trace, "O")
        qkv_value = self._rescale(self.rs, t["qkv_rem"], e2, T, d, qkv_cl, s.scale1, trace, "qkv")
        # ---- softmax x V (test/llm.cu:369-388); V is stored transposed [L][d][T]
        soft, ssize = self._fr(t["softmax"])
        soft_keep = self._clone(soft, ssize * 32)
        xv, _ = self._fr(t["xv_q"])
        e3 = self._draw(log2ceil(L * T))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            soft_cl, xv_cl, _, _ = host.prove_matmul(ctx, soft, xv, L, T, d, T, e2, e3, qkv_value)
        e2, e3 = reassemble_vectors(e2, e3, lT, lT, ld)
        skip_point = list(e3)                                   # point of the claim on V^T
        if self._open(soft_keep, ssize, e2, T, trace)["result"] != soft_cl:
            raise ProofError("softmax x V: opening of the softmax output disagrees")
        self._release(soft, xv)
        # ---- softmax rounding relation (test/llm.cu:391-409):
        #      2 * scale * e - (2 o - 1) * rowsum(e) must lie in [0, softmax_len)
        e_out, _ = self._fr(t["exp_out"])
        resid = self._alloc(ssize * 32)
        tmp = self._alloc(ssize * 32)
        consts = ctx.fr_upload([2 * s.scale1, 2, -1])
        ctx.fr_binary("scale", e_out, consts, resid, ssize)                 # e * 2 * scale
        ctx.fr_binary("scale", soft_keep, consts.at(32), soft_keep, ssize)  # 2 o
        ctx.fr_binary("add_scalar", soft_keep, consts.at(64), soft_keep, ssize)  # 2 o - 1
        ctx.fr_rowsum(e_out, tmp, ssize // T, T)
        ctx.fr_binary("mul", soft_keep, tmp, soft_keep, ssize)
        ctx.fr_binary("sub", resid, soft_keep, resid, ssize)
        e1 = self._draw(log2ceil(ssize))
        trace.lookups += 1
        with self._phase(trace, "lookup"):
            self.softmax_range.prove(resid, ssize, tmp, e1, table=self.table, msm_size=T)
        self._open(e_out, ssize, e1, T, trace)
        self._release(resid, tmp, soft_keep)
        consts.free()
        # ---- exp mapping lookup (test/llm.cu:412-422)
        e_in, _ = self._fr(t["exp_in"])
        e1 = self._draw(log2ceil(ssize))
        work, Abuf = self._alloc(ssize * 32), self._alloc(ssize * 32)
        trace.lookups += 1
        with self._phase(trace, "lookup"):
            lookup_value, _ = self.exp.prove_pairs(e_in, e_out, ssize, work, Abuf, e1, table=self.table, msm_size=T)
        exp_in_value = self._open(e_in, ssize, e1, T, trace)["result"]
        exp_out_value = self._open(e_out, ssize, e1, T, trace)["result"]
        if lookup_value != (exp_in_value + exp_out_value * self.exp.r) % R:
            raise ProofError("exp: lookup claim disagrees with the two openings")
        self._release(e_in, e_out, work, Abuf)
        # ---- scores (test/llm.cu:425-437): quotient evaluated, remainder opened, scale 2^22
        sc, _ = self._fr(t["scores_q"])
        score_value = ctx.fr_eval(sc, ssize, e1)
        sc_rem, _ = self._fr(t["scores_rem"])
        score_value = (score_value * s.scale3 + self._open(sc_rem, ssize, e1, T, trace)["result"]) % R
        self._release(sc, sc_rem)
        # ---- Q K^T (test/llm.cu:440-452)
        xq, _ = self._fr(t["xq_q"])
        xk, _ = self._fr(t["xk_q"])
        e2 = self._draw(log2ceil(L * d))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            q_cl, k_cl, _, _ = host.prove_matmul(ctx, xq, xk, L, T, T, d, e1, e2, score_value)
        e1, e2 = reassemble_vectors(e1, e2, lT, ld, lT)
        self._release(xq, xk)
        # ---- Q projection, K projection (test/llm.cu:455-513)
        n1, nsize = self._fr(t["norm1_q"])
        q_value = self._rescale(self.rs, t["xq_rem"], e1, d, d, q_cl, s.scale1, trace, "xq")
        out1, e1, _ = self._matmul_open_w(None, t["W_Q"], T, d, d, e1, q_value, trace, "Q", keep_A=self._clone(n1, nsize * 32))
        k_value = self._rescale(self.rs, t["xk_rem"], e2, d, d, k_cl, s.scale1, trace, "xk")
        out2, e2, _ = self._matmul_open_w(None, t["W_K"], T, d, d, e2, k_value, trace, "K", keep_A=self._clone(n1, nsize * 32))
        # ---- V projection, proven transposed: V^T = W_V * normOut^T (test/llm.cu:516-545)
        v_value = self._rescale(self.rs, t["xv_rem"], skip_point, d, d, xv_cl, s.scale1, trace, "xv")
        WV, wsize = self._fr(t["W_V"])
        WV_keep = self._clone(WV, wsize * 32)
        n1b = self._clone(n1, nsize * 32)
        e3 = self._draw(log2ceil(L * d))
        trace.matmuls += 1
        with self._phase(trace, "matmul"):
            wv_cl, out3, _, _ = host.prove_matmul(ctx, WV, n1b, L, d, T, d, skip_point, e3, v_value)
        skip_point, e3 = reassemble_vectors(skip_point, e3, ld, ld, lT)
        if self._open(WV_keep, wsize, skip_point, d, trace)["result"] != wv_cl:
            raise ProofError("V: opening of W_V disagrees with the sumcheck claim")
        self._release(WV, WV_keep, n1b)
        # ---- three claims on the first norm output become one (test/llm.cu:548-556)
        point = self._draw(log2ceil(nsize))
        with self._phase(trace, "combine"):
            norm1_value, _ = host.combine_claims(ctx, n1, nsize, [out1, out2, out3], [e1, e2, e3], point)
        self._release(n1)
        # ---- first norm (test/llm.cu:559-601) and the final opening of the layer input (:604-609)
        x_cl, e1, inp_keep = self._norm(t, "1", t["input"], norm1_value, point, trace)
        final = self._open(inp_keep, size, e1, d, trace)["result"]
        if final != x_cl:
            raise ProofError("input: opening disagrees with the Hadamard sumcheck claim")
        self._release(inp_keep)
        trace.values["input"] = final
        trace.values["input_point"] = e1
        return trace
