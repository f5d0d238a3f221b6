"""Blob formats (CPU) and the commit-all-tensors driver (GPU)."""
import numpy as np
import pytest

from oracle import bn254, cport
from oracle import protocols as pr


def test_blob_roundtrip(tmp_path):
    from grape_b200 import io
    t = np.arange(-5, 7, dtype=np.int32)
    io.save_blob(tmp_path / "W" / "x-0.bin", t)
    assert (io.load_int32(tmp_path / "W" / "x-0.bin") == t).all()
    rec = np.arange(48, dtype=np.uint32).reshape(2, 24)
    io.save_blob(tmp_path / "c.bin", rec)
    assert (io.load_commitments(tmp_path / "c.bin") == rec).all()
    io.save_blob(tmp_path / "bad.bin", np.zeros(25, dtype=np.uint32))
    with pytest.raises(ValueError):
        io.load_commitments(tmp_path / "bad.bin")
    table = np.zeros((256, 3, 16), dtype=np.uint32)
    io.save_blob(tmp_path / "points.bin", table[:, :2])           # too short, like the reference's ppgen output
    with pytest.raises(ValueError):
        io.load_points_bin(tmp_path / "points.bin", 3)
    io.save_blob(tmp_path / "points.bin", table)
    assert io.load_points_bin(tmp_path / "points.bin", 3).shape == (256, 3, 16)


def test_pad_rows_matches_reference_rule():
    from grape_b200 import commit_pipeline as cp
    t = np.arange(12, dtype=np.int32)
    assert cp.pad_rows(t, 4) is t
    out = cp.pad_rows(t, 3).reshape(4, 4)
    assert (out[:, :3] == t.reshape(4, 3)).all() and (out[:, 3] == 0).all()
    lists = cp.file_lists(2048)
    assert [k for k, _, _ in lists] == ["W", "R", "Q"] and ("down-", 11008) in lists[0][2]


@pytest.mark.gpu
def test_points_bin_export_and_commit_all(gctx, tmp_path):
    import grape_b200 as g
    from grape_b200 import commit_pipeline as cp, io
    gens = bn254.make_generators(64, seed=8)
    gj = g.encode_jacobian(gens)
    exported = io.export_points_bin(gctx, gj)
    assert exported.tobytes() == cport.table_build(gj).tobytes()      # the reference's points.bin content
    io.save_blob(tmp_path / "points.bin", exported)
    # a Hyrax table wrapping that file commits like the native one
    d_points = gctx.upload(io.load_points_bin(tmp_path / "points.bin", 64))
    import ctypes as C
    h = C.c_void_p()
    gctx._check(gctx.lib.grape_table_from_reference(gctx.handle, d_points.ptr, 64, C.byref(h)))
    rng = np.random.default_rng(4)
    lists = [("W", "comW", [("up-", 4), ("down-", 3)])]               # N = 4 (wd 64) and N = 3 -> padded to 4
    for name, n in lists[0][2]:
        for b in range(2):
            io.save_blob(tmp_path / "W" / f"{name}{b}.bin", rng.integers(-2**31, 2**31, size=n * 16 * 3, dtype=np.int64).astype(np.int32))
    table = g.GeneratorTable(gctx, gj, 8, 1)
    secs = cp.commit_all(gctx, table, tmp_path, batches=2, lists=lists)
    assert "W" in secs
    for name, n in lists[0][2]:
        for b in range(2):
            t = io.load_int32(tmp_path / "W" / f"{name}{b}.bin")
            padded = cp.pad_rows(t, n)
            want = pr.commit_rows([int(x) for x in padded], 64, gens)
            got = io.load_commitments(tmp_path / "comW" / f"{name}{b}.bin")
            assert g.decode_jacobian(got) == want
            # same rows through the reference-layout table
            d = gctx.upload(padded)
            out = gctx.alloc(got.shape[0] * 96)
            gctx._check(gctx.lib.grape_commit_i32(gctx.handle, h, d.ptr, padded.size, 64, 32, out.ptr))
            assert gctx.download(out, got.nbytes).tobytes() == got.tobytes()
    gctx.lib.grape_table_destroy(h)
    table.close()


def test_rmsnorm_factor_is_the_integer_rsqrt_of_the_model():
    """The synthesised layers derive their RMSNorm factor as the model does (zzllama/llama/model.py:204,
    221-226): rms = round(scale / sqrt(mean((x/scale)^2) + eps)).  The integer square root must agree
    with a float64 evaluation to within one unit of the quantisation step, on inputs of the scale the
    benchmark uses, and the two rescales that follow must be exact."""
    import numpy as np
    from grape_b200 import layer_full
    from grape_b200.layer import round_div
    rng = np.random.default_rng(4)
    scale = 1 << 16
    x = rng.integers(-(1 << 13), 1 << 13, size=(2, 9, 4096)).astype(np.int64)
    x[0, 0] = 0                       # an all-zero token: the factor is scale / sqrt(eps)
    x[0, 1] = (1 << 20)               # a large-magnitude token
    r = layer_full.rms_factor(x, scale)
    xr = x.astype(np.float64) / scale
    f = scale / np.sqrt((xr ** 2).mean(-1) + 1e-5)
    assert np.all(np.abs(r - f) <= 1.0)
    assert r[0, 0] == round(scale / np.sqrt(1e-5))
    shape = layer_full.LayerShape(layer_num=1, tokens=4, dim=64, ffn=96, scale1=256, scale2=512, swiglu_low=-256,
                                  swiglu_len=512, npoints=64, scale3=1 << 9, exp_low=-511, exp_len=512, softmax_len=512)
    t = layer_full.synthesize_layer(shape, seed=3, x_range=256, w_std=8.0)
    inp = t["input"].astype(np.int64)
    assert np.array_equal(t["rms1"].reshape(1, 4), layer_full.rms_factor(inp, 256))
    prod = t["rms1"].astype(np.int64) * t["wnorm1"].astype(np.int64).reshape(1, 1, 64)
    assert np.array_equal(prod, t["rmsw1_q"].astype(np.int64) * 256 + t["rmsw1_rem"])
    assert np.array_equal(inp * t["rmsw1_q"], t["norm1_q"].astype(np.int64) * 256 + t["norm1_rem"])
    assert np.abs(t["rmsw1_rem"]).max() <= 128 and np.abs(t["norm1_rem"]).max() <= 128
