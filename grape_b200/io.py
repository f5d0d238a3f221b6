"""On-disk formats of the reference, as raw little-endian blobs (src/ioutils.cu:3-103):

  points.bin        affine table, 256 rows x n generators x 64 B, row w = w * G_i   (test/ppgen.cu:23)
  cpu_points.bin    generators as Jacobian records, 96 B each                      (test/ppgen.cu:24)
  data/{W,Q,R}/<name>-<batch>.bin   int32 tensors, the layers of one batch appended (zzllama/llama/model.py:46-63)
  data/com{W,Q,R}/<name>-<batch>.bin  row commitments, 96 B Jacobian records         (test/commit.cu:65-66)
  data/table/*.bin  int32 mapping tables                                            (src/tlookup.cu:355-358)
"""
from __future__ import annotations

from pathlib import Path

import numpy as np


def save_blob(path, arr: np.ndarray):
    """``savebin``: the bytes of the array, nothing else."""
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    np.ascontiguousarray(arr).tofile(str(path))


def load_int32(path) -> np.ndarray:
    """``load_data``: a whole file of int32 values."""
    return np.fromfile(str(path), dtype="<i4")


def load_points_bin(path, n_gens: int) -> np.ndarray:
    """points.bin -> uint32[256, n_gens, 16]; raises if the file is shorter (the reference's ppgen
    writes fewer bytes than its readers expect, test/ppgen.cu:17 versus test/commit.cu:28-29)."""
    raw = np.fromfile(str(path), dtype="<u4")
    need = 256 * n_gens * 16
    if raw.size < need:
        raise ValueError(f"{path}: {raw.size * 4} bytes, a table of {n_gens} generators needs {need * 4}")
    return raw[:need].reshape(256, n_gens, 16)


def load_generators(path, n_gens: int) -> np.ndarray:
    """cpu_points.bin -> uint32[n_gens, 24] Jacobian records."""
    raw = np.fromfile(str(path), dtype="<u4", count=n_gens * 24)
    if raw.size < n_gens * 24:
        raise ValueError(f"{path}: too short for {n_gens} generators")
    return raw.reshape(n_gens, 24)


def load_commitments(path) -> np.ndarray:
    raw = np.fromfile(str(path), dtype="<u4")
    if raw.size % 24:
        raise ValueError(f"{path}: not a whole number of 96-byte records")
    return raw.reshape(-1, 24)


def export_points_bin(ctx, gens_jacobian: np.ndarray) -> np.ndarray:
    """The reference's 256-row table for these generators (what test/ppgen.cu writes), computed with
    the library's table builder: uint32[256, n, 16] with row 0 = infinity."""
    from .host import GeneratorTable
    n = gens_jacobian.shape[0]
    t = GeneratorTable(ctx, gens_jacobian, window_bits=9, n_windows=1)   # magnitudes 1..256
    rows = ctx.download(ctx.lib.grape_table_data(t.handle), 255 * n * 64).reshape(255, n, 16)
    out = np.zeros((256, n, 16), dtype=np.uint32)
    out[1:] = rows
    t.close()
    return out
