"""The feed-forward half of the layer driver (the call order of the reference's test/llm.cu:73-262)
on self-consistent synthetic tensors: every junction value equals the oracle's."""
import numpy as np
import pytest

from oracle import bn254, cport, layer as olayer

pytestmark = pytest.mark.gpu


def test_ffn_block_matches_oracle(gctx):
    import grape_b200 as g
    from grape_b200 import layer, workloads as wl
    shape = layer.FFNShape(layer_num=2, tokens=16, dim=32, ffn=48, scale1=256, scale2=512, swiglu_low=-256,
                           swiglu_len=512, npoints=64)
    t = layer.synthesize_ffn(shape, seed=11, x_range=64, w_std=8.0)
    assert t["gate_q"].min() >= -256 and t["gate_q"].max() < 256
    n_gens = shape.ffn_pad * 16
    gens_j = wl.make_generators(gctx, n_gens, seed=77)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    gctx.seed(2024)
    prover = layer.FFNProver(gctx, shape, table, gens_j[0], t["swiglu_table"])
    trace = prover.prove(t)
    assert trace.opens == 10 and trace.lookups == 5 and trace.matmuls == 3
    assert all(trace.values[k] != 0 for k in ("down_out", "upSilu", "up_out", "gate_out"))
    # oracle walk with the same stream
    gens = g.decode_jacobian(gens_j)
    ctable = cport.table_build(gens_j)

    def msm_fn(scalars, points):
        enc = np.frombuffer(bn254.fr_vec_to_bytes(scalars), dtype=np.uint32).reshape(-1, 8)
        rec = cport.commit_fr(enc, len(scalars), ctable[:, :len(scalars)].copy())
        return bn254.jacobian_from_bytes(rec[0].tobytes())

    flat = {k: v.reshape(-1).tolist() for k, v in t.items()}
    want = olayer.prove_ffn(flat, shape, gens, bn254.SplitMix64(2024), msm_fn)
    for key in ("skip", "down_out", "upSilu", "silu_at_e2", "up_out", "gate_out", "normOutSecond",
                "normOutSecond_point", "skip_point"):
        assert trace.values[key] == want[key], key
    table.close()


def test_ffn_block_rejects_inconsistent_remainder(gctx):
    """A remainder that does not belong to the committed product breaks a round check downstream."""
    import grape_b200 as g
    from grape_b200 import layer, workloads as wl
    shape = layer.FFNShape(layer_num=1, tokens=16, dim=32, ffn=48, scale1=256, scale2=512, swiglu_low=-256,
                           swiglu_len=512, npoints=64)
    t = layer.synthesize_ffn(shape, seed=12, x_range=64, w_std=8.0)
    t["down_rem"] = t["down_rem"].copy()
    t["down_rem"].reshape(-1)[5] += 1 if t["down_rem"].reshape(-1)[5] < 100 else -1
    gens_j = wl.make_generators(gctx, shape.ffn_pad * 16, seed=78)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    gctx.seed(1)
    prover = layer.FFNProver(gctx, shape, table, gens_j[0], t["swiglu_table"])
    with pytest.raises(g.GrapeError):
        prover.prove(t)
    table.close()


def test_whole_layer_matches_oracle(gctx):
    """FFN half, both RMSNorms, attention (softmax relation, exp lookup, score / Q / K / V matmuls)."""
    import grape_b200 as g
    from grape_b200 import layer_full, workloads as wl
    shape = layer_full.LayerShape(layer_num=2, tokens=16, dim=32, ffn=48, scale1=256, scale2=512, swiglu_low=-256,
                                  swiglu_len=512, npoints=64, scale3=1 << 9, exp_low=-511, exp_len=512,
                                  softmax_len=512)
    t = layer_full.synthesize_layer(shape, seed=5, x_range=512, w_std=12.0)
    assert np.abs(t["xq_q"]).max() > 0 and np.abs(t["qkv_q"]).max() > 0 and t["exp_in"].min() < 0
    gens_j = wl.make_generators(gctx, shape.ffn_pad * 16, seed=79)
    table = g.GeneratorTable(gctx, gens_j, 8, 1)
    gctx.seed(31337)
    prover = layer_full.LayerProver(gctx, shape, table, gens_j[0], t["swiglu_table"], t["exp_table"])
    trace = prover.prove_layer(t)
    assert trace.matmuls == 11 and trace.lookups == 16  # the reference's 11 matmul sumchecks, 14 range + 2 mapping lookups
    gens = g.decode_jacobian(gens_j)
    ctable = cport.table_build(gens_j)

    def msm_fn(scalars, points):
        enc = np.frombuffer(bn254.fr_vec_to_bytes(scalars), dtype=np.uint32).reshape(-1, 8)
        rec = cport.commit_fr(enc, len(scalars), ctable[:, :len(scalars)].copy())
        return bn254.jacobian_from_bytes(rec[0].tobytes())

    flat = {k: v.reshape(-1).tolist() for k, v in t.items()}
    want = olayer.prove_layer(flat, shape, gens, bn254.SplitMix64(31337), msm_fn)
    for key in want:
        assert trace.values[key] == want[key], key
    prover.release_pool()
    table.close()
