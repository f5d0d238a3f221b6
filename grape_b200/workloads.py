"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference proves real LLaMA-2-7B tensors dumped to disk; those files are not distributable, so
the configurations are stood in for by random-init tensors of the same shapes: weights drawn from
N(0, 0.02), scaled by 2^16, rounded and clipped (the quantisation the reference's data producer
applies, zzllama/llama/model.py:22-63), and generators G_i = [rho_i] * (1, 2) with seeded rho_i.
"""
from __future__ import annotations

import numpy as np

from .host import Context, GeneratorTable, commit_fr, encode_jacobian

LLAMA_DIM = 4096
LLAMA_FFN = 11008
#: (rows, cols) of the seven weight matrices of one LLaMA-2-7B decoder layer (q, k, v, o, gate, up, down)
LLAMA_LAYER_WEIGHTS = [(LLAMA_DIM, LLAMA_DIM)] * 4 + [(LLAMA_FFN, LLAMA_DIM)] * 2 + [(LLAMA_DIM, LLAMA_FFN)]


def quantised_normal(rng: np.random.Generator, n: int, std: float = 0.02, scale: int = 1 << 16,
                     lo: int = -(1 << 15), hi: int = (1 << 15) - 1, out: np.ndarray | None = None) -> np.ndarray:
    """clip(round(N(0, std) * scale), lo, hi) as int32, generated in slices to bound memory."""
    if out is None:
        out = np.empty(n, dtype=np.int32)
    step = 1 << 24
    for s in range(0, n, step):
        e = min(n, s + step)
        x = rng.standard_normal(e - s, dtype=np.float32)
        np.multiply(x, std * scale, out=x)
        np.rint(x, out=x)
        np.clip(x, lo, hi, out=x)
        out[s:e] = x.astype(np.int32)
    return out


def layer_weight_elements() -> int:
    return sum(r * c for r, c in LLAMA_LAYER_WEIGHTS)


def make_generators(ctx: Context, n: int, seed: int) -> np.ndarray:
    """n generators [rho_i] * (1, 2) as uint32[n, 24] Jacobian records, computed on the GPU with the
    library's own fixed-base commitment (one row per generator over the single base point)."""
    base = GeneratorTable(ctx, encode_jacobian([(1, 2)]), window_bits=8, n_windows=32)
    ctx.seed(seed)
    rho = ctx.random_fr(n)
    d_rho = ctx.upload(rho)
    d_out = ctx.alloc(n * 96)
    commit_fr(ctx, base, d_rho, n, 1, d_out)
    gens = ctx.download(d_out, n * 96).reshape(n, 24)
    base.close()
    d_rho.free()
    d_out.free()
    return gens


def exact_matmul_cuda(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """[l, n, k] x [l, m, k]^T for int64 arrays, computed exactly on the GPU in float64 (all
    partial sums of the synthetic tensors stay far below 2^53).  Data preparation only: this is
    the stand-in for the model's forward pass that produced the reference's dumps."""
    import torch
    ta = torch.from_numpy(np.ascontiguousarray(a)).cuda().double()
    tb = torch.from_numpy(np.ascontiguousarray(b)).cuda().double()
    r = torch.matmul(ta, tb.transpose(1, 2)).round().long().cpu().numpy()
    del ta, tb
    torch.cuda.empty_cache()
    return r


#: the standard BLS12-381 G1 generator as a 144-byte Jacobian record (X|Y|1, Montgomery limbs, radix 2^384)
_BLS_P = 0x1A0111EA397FE69A4B1BA7B6434BACD764774B84F38512BF6730D2A0F6B0F6241EABFFFEB153FFFFB9FEFFFFFFFFAAAB
_BLS_G1 = (
    0x17F1D3A73197D7942695638C4FA9AC0FC3688C4F9774B905A14E3A3F171BAC586C55E83FF97A1AEFFB3AF00ADB22C6BB,
    0x08B3F481E3AAA0F1A09E30ED741D8AE4FCF5E095D5D00AF600DB18CB2C04B3EDD03CC744A2888AE40CAA232946C5E7E1,
)


def make_generators_bls12_381(ctx: Context, n: int, seed: int) -> np.ndarray:
    """n BLS12-381 generators [rho_i] * G1 as uint32[n, 36] Jacobian records, computed on the GPU
    with the library's own fixed-base commitment over the single standard generator.  rho_i are the
    seeded stream's 32-byte draws read as BLS12-381 scalar-field residues."""
    rec = b"".join(((c << 384) % _BLS_P).to_bytes(48, "little") for c in (_BLS_G1[0], _BLS_G1[1], 1))
    base = GeneratorTable(ctx, np.frombuffer(rec, dtype=np.uint32).reshape(1, 36), window_bits=8, n_windows=32,
                          curve="bls12_381")
    ctx.seed(seed)
    rho = ctx.random_fr(n)
    d_rho = ctx.upload(rho)
    d_out = ctx.alloc(n * 144)
    commit_fr(ctx, base, d_rho, n, 1, d_out)
    gens = ctx.download(d_out, n * 144).reshape(n, 36)
    base.close()
    d_rho.free()
    d_out.free()
    return gens
