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
    return _ffn_with_state(t, shape, gens, draw, msm_fn, None)


def _ffn_with_state(t, shape, gens, draw, msm_fn, state):
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
    if state is not None:  # the whole-layer walk constructs two more lookup objects before proving
        state.update({"c": c, "rs": rs, "softmax_alpha": draw.next_fr(), "exp_alpha": draw.next_fr(),
                      "exp_r": draw.next_fr()})
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


def prove_layer(t, shape, gens, draw: bn254.SplitMix64, msm_fn=None):
    """The whole layer walk (test/llm.cu:73-611), mirror of ``grape_b200/layer_full.py``."""
    L, T, d, F = shape.layer_num, shape.tokens, shape.dim, shape.ffn
    lT, ld = pr.log2ceil(T), pr.log2ceil(d)
    size = L * T * d
    G = gens[0]
    fr = lambda xs: [int(x) % R for x in xs]
    # random objects in construction order: c, rs, swiglu_rs, swiglu (alpha, r), softmax range, exp (alpha, r)
    state = {}
    values = _ffn_with_state(t, shape, gens, draw, msm_fn, state)
    c, rs = state["c"], state["rs"]

    def open_(tensor, n, e, N):
        d_blind = draw.fr_vec((1 << pr.log2ceil(N)) * 16)
        return pr.hyrax_open(tensor, e, c, n, N, L, gens, G, d_blind, msm_fn)

    def rescale(rem, e, open_N, q_claim, scale, name):
        rem = fr(rem)
        u = draw.fr_vec(pr.log2ceil(len(rem)))
        got = rs.prove(rem, e, u)
        assert open_(rem, len(rem), e, open_N)["result"] == got["claim"], name
        values[name] = (q_claim * scale + got["claim"]) % R
        return values[name]

    def matmul_open_w(A, W_ints, N, M, K, u, claim):
        W = fr(W_ints)
        v = draw.fr_vec(pr.log2ceil(K * L))
        a_cl, w_cl, _, _ = pr.prove_matmul(A, W, L, N, M, K, u, v, claim)
        u2, v2 = pr.reassemble_vectors(u, v, pr.log2ceil(N), pr.log2ceil(K), pr.log2ceil(M))
        assert open_(W, len(W), v2, K)["result"] == w_cl
        return a_cl, u2, v2

    def norm(tag, x_ints, value, e3):
        value = rescale(t[f"norm{tag}_rem"], e3, d, value, shape.scale1, f"norm{tag}")
        x, rmsw = fr(x_ints), fr(t[f"rmsw{tag}_q"])
        e1 = draw.fr_vec(pr.log2ceil(size))
        x_cl, rmsw_cl, _, _ = pr.prove_elemul(x, rmsw, L, T, d, e3, e1, value)
        rmsw_value = rescale(t[f"rmsw{tag}_rem"], e1, d, rmsw_cl, shape.scale1, f"rmsw{tag}")
        e3n = draw.fr_vec(pr.log2ceil(L))
        rms, wn = fr(t[f"rms{tag}"]), fr(t[f"wnorm{tag}"])
        rms_cl, wn_cl, _, _ = pr.prove_matmul(rms, wn, L, T, d, 1, e1, e3n, rmsw_value)
        e2, e3n = pr.reassemble_vectors(e1, e3n, lT, 0, ld)
        assert open_(wn, len(wn), e3n, d // 16)["result"] == wn_cl
        assert open_(rms, len(rms), e2, T // 16)["result"] == rms_cl
        return x_cl, e1, x

    softmax_range = pr.LookupRange(0, shape.softmax_len, state["softmax_alpha"])
    exp = pr.LookupRangeMapping(shape.exp_low, shape.exp_len, [int(x) for x in t["exp_table"]], state["exp_alpha"],
                                state["exp_r"])
    skip_value, skip_point = values["skip"], values["skip_point"]
    x_cl, e1, skip_t = norm("2", t["skip"], values["normOutSecond"], values["normOutSecond_point"])
    e2 = draw.fr_vec(pr.log2ceil(size))
    skip_value, _ = pr.combine_claims(skip_t, [skip_value, x_cl], [skip_point, e1], e2, size)
    input_value = open_(fr(t["input"]), size, e2, d)["result"]
    atten_value = rescale(t["atten_rem"], e2, d, (skip_value - input_value) % R, shape.scale1, "atten_out")
    qkv_cl, e2, _ = matmul_open_w(fr(t["qkv_q"]), t["W_O"], T, d, d, e2, atten_value)
    qkv_value = rescale(t["qkv_rem"], e2, d, qkv_cl, shape.scale1, "qkv")
    soft, xv = fr(t["softmax"]), fr(t["xv_q"])
    ssize = len(soft)
    e3 = draw.fr_vec(pr.log2ceil(L * T))
    soft_cl, xv_cl, _, _ = pr.prove_matmul(soft, xv, L, T, d, T, e2, e3, qkv_value)
    e2, e3 = pr.reassemble_vectors(e2, e3, lT, lT, ld)
    skip_point = list(e3)
    assert open_(soft, ssize, e2, T)["result"] == soft_cl
    e_out = fr(t["exp_out"])
    rowsum = [sum(e_out[r * T:(r + 1) * T]) % R for r in range(ssize // T)]
    resid = [(2 * shape.scale1 * e_out[i] - (2 * soft[i] - 1) * rowsum[i // T]) % R for i in range(ssize)]
    e1 = draw.fr_vec(pr.log2ceil(ssize))
    u = draw.fr_vec(pr.log2ceil(ssize))
    softmax_range.prove(resid, e1, u)
    open_(e_out, ssize, e1, T)
    e_in = fr(t["exp_in"])
    e1 = draw.fr_vec(pr.log2ceil(ssize))
    u = draw.fr_vec(pr.log2ceil(ssize))
    got = exp.prove_pairs(e_in, e_out, e1, u)
    exp_in_value = open_(e_in, ssize, e1, T)["result"]
    exp_out_value = open_(e_out, ssize, e1, T)["result"]
    assert got["claim"] == (exp_in_value + exp_out_value * exp.r) % R
    score_value = pr.tensor_eval(fr(t["scores_q"]), e1)
    score_value = (score_value * shape.scale3 + open_(fr(t["scores_rem"]), ssize, e1, T)["result"]) % R
    e2 = draw.fr_vec(pr.log2ceil(L * d))
    q_cl, k_cl, _, _ = pr.prove_matmul(fr(t["xq_q"]), fr(t["xk_q"]), L, T, T, d, e1, e2, score_value)
    e1, e2 = pr.reassemble_vectors(e1, e2, lT, ld, lT)
    n1 = fr(t["norm1_q"])
    q_value = rescale(t["xq_rem"], e1, d, q_cl, shape.scale1, "xq")
    out1, e1, _ = matmul_open_w(n1, t["W_Q"], T, d, d, e1, q_value)
    k_value = rescale(t["xk_rem"], e2, d, k_cl, shape.scale1, "xk")
    out2, e2, _ = matmul_open_w(n1, t["W_K"], T, d, d, e2, k_value)
    v_value = rescale(t["xv_rem"], skip_point, d, xv_cl, shape.scale1, "xv")
    WV = fr(t["W_V"])
    e3 = draw.fr_vec(pr.log2ceil(L * d))
    wv_cl, out3, _, _ = pr.prove_matmul(WV, n1, L, d, T, d, skip_point, e3, v_value)
    skip_point, e3 = pr.reassemble_vectors(skip_point, e3, ld, ld, lT)
    assert open_(WV, len(WV), skip_point, d)["result"] == wv_cl
    point = draw.fr_vec(pr.log2ceil(len(n1)))
    norm1_value, _ = pr.combine_claims(n1, [out1, out2, out3], [e1, e2, e3], point, len(n1))
    x_cl, e1, inp = norm("1", t["input"], norm1_value, point)
    final = open_(inp, size, e1, d)["result"]
    assert final == x_cl
    values["input"] = final
    values["input_point"] = e1
    return values
