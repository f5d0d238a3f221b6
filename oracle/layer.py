"""CPU oracle, part 4: the feed-forward half of the reference's layer driver (test/llm.cu:73-262)
restated with the oracle's protocol functions.  TEST INFRASTRUCTURE ONLY.

Same walk, same junction checks and the same order of random draws as
``grape_b200/layer.py``; used at small shapes to check the values at every junction.
"""
from __future__ import annotations

from . import bn254
from . import protocols as pr
from .bn254 import R


def prove_ffn(t, shape, gens, draw: bn254.SplitMix64, msm_fn=None):
    """t: dict of integer lists (flattened tensors); shape: object with layer_num, tokens, dim, ffn,
    scale1, scale2, swiglu_low, swiglu_len.  Returns the dict of junction values."""
    L, T, d, F = shape.layer_num, shape.tokens, shape.dim, shape.ffn
    Fp = 1 << pr.log2ceil(F)
    lT, ld, lF = pr.log2ceil(T), pr.log2ceil(d), pr.log2ceil(F)
    G = gens[0]
    fr = lambda xs: [int(x) % R for x in xs]
    c = draw.next_fr()
    rs = pr.LookupRange(-(shape.scale1 // 2), shape.scale1, draw.next_fr())
    swiglu_rs = pr.LookupRange(-(shape.scale2 // 2), shape.scale2, draw.next_fr())
    swiglu = pr.LookupRangeMapping(shape.swiglu_low, shape.swiglu_len, [int(x) for x in t["swiglu_table"]],
                                   draw.next_fr(), draw.next_fr())
    values = {}

    def open_(tensor, size, e, N):
        d_blind = draw.fr_vec((1 << pr.log2ceil(N)) * 16)
        return pr.hyrax_open(tensor, e, c, size, N, L, gens, G, d_blind, msm_fn)

    def rescale(lk, rem, e, open_N, q_claim, scale, name):
        rem = fr(rem)
        u = draw.fr_vec(pr.log2ceil(len(rem)))
        got = lk.prove(rem, e, u, inner=F, inner_pad=Fp)
        proof = open_(rem, len(rem), e, open_N)
        assert proof["result"] == got["claim"], name
        values[name] = (q_claim * scale + got["claim"]) % R
        return values[name]

    out = fr(t["output"])
    size = len(out)
    e1 = draw.fr_vec(pr.log2ceil(size))
    proof = open_(out, size, e1, size // L // T)
    down_out_value = pr.tensor_eval(fr(t["down_q"]), e1)
    values["skip"] = (proof["result"] - down_out_value) % R
    values["skip_point"] = list(e1)
    down_out_value = rescale(rs, t["down_rem"], e1, size // L // T, down_out_value, shape.scale1, "down_out")
    W = fr(t["W_down"])
    e2 = draw.fr_vec(pr.log2ceil(F * L))
    a_cl, b_cl, _, _ = pr.prove_matmul(fr(t["upsilu_q"]), W, L, T, d, F, e1, e2, down_out_value)
    e1, e2 = pr.reassemble_vectors(e1, e2, lT, lF, ld)
    assert open_(W, len(W), e2, F)["result"] == b_cl
    upsilu_value = rescale(rs, t["upsilu_rem"], e1, F, a_cl, shape.scale1, "upSilu")
    up, silu = fr(t["up_q"]), fr(t["silu"])
    e2 = draw.fr_vec(pr.log2ceil(len(up)))
    up_cl, silu_cl, _, _ = pr.prove_elemul(up, silu, L, T, F, e1, e2, upsilu_value)
    values["silu_at_e2"] = silu_cl
    gate = fr(t["gate_q"])
    e1 = draw.fr_vec(pr.log2ceil(len(gate)))
    u = draw.fr_vec(pr.log2ceil(len(gate)))
    got = swiglu.prove_pairs(gate, silu, e1, u, inner=F, inner_pad=Fp)
    gate_out_value = open_(gate, len(gate), e1, F)["result"]
    silu_open = open_(silu, len(silu), e1, F)["result"]
    assert got["claim"] == (gate_out_value + silu_open * swiglu.r) % R
    up_out_value = rescale(rs, t["up_rem"], e2, F, up_cl, shape.scale1, "up_out")
    x = fr(t["x"])
    W = fr(t["W_up"])
    e3 = draw.fr_vec(pr.log2ceil(d * L))
    n1, w_cl, _, _ = pr.prove_matmul(x, W, L, T, F, d, e2, e3, up_out_value)
    e2, e3 = pr.reassemble_vectors(e2, e3, lT, ld, lF)
    assert open_(W, len(W), e3, d)["result"] == w_cl
    gate_out_value = rescale(swiglu_rs, t["gate_rem"], e1, F, gate_out_value, shape.scale2, "gate_out")
    W = fr(t["W_gate"])
    e3 = draw.fr_vec(pr.log2ceil(d * L))
    n2, w_cl, _, _ = pr.prove_matmul(x, W, L, T, F, d, e1, e3, gate_out_value)
    e1, e3 = pr.reassemble_vectors(e1, e3, lT, ld, lF)
    assert open_(W, len(W), e3, d)["result"] == w_cl
    e3 = draw.fr_vec(pr.log2ceil(d * L * T))
    value, _ = pr.combine_claims(x, [n1, n2], [e2, e1], e3, d * L * T)
    values["normOutSecond"] = value
    values["normOutSecond_point"] = e3
    return values
