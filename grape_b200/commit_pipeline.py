"""Commit-all-tensors driver: the flow of the reference's test/commit.cu (:39-171) — for every
tensor file of a batch, load int32 data, pad rows to a power of two, commit rows of N*16 scalars,
write the commitments.  The file lists and row lengths are the reference's.
"""
from __future__ import annotations

import time
from pathlib import Path

import numpy as np

from . import io
from .host import COM_SCALE, Context, GeneratorTable, commit_i32_host


def file_lists(input_tokens: int = 2048):
    """(directory, commitment directory, [(name, N)]) as in test/commit.cu:39-136."""
    W = [("down-", 11008), ("up-", 4096), ("gate-", 4096), ("NormSecond-", 4096 // COM_SCALE),
         ("NormFirst-", 4096 // COM_SCALE), ("O-", 4096), ("K-", 4096), ("Q-", 4096), ("V-", 4096)]
    R = [("down_out-", 4096), ("up_out-", 11008), ("gate_out-", 11008), ("upSilu-", 11008), ("atten_out-", 4096),
         ("normOutFirst-", 4096), ("normOutSecond-", 4096), ("qkv-", 4096), ("rmswFirst-", 4096),
         ("rmswSecond-", 4096), ("scores-", input_tokens), ("xk-", 4096), ("xv-", 4096), ("xq-", 4096)]
    Q = [("exp_input-", input_tokens), ("exp_output-", input_tokens), ("softmax_output-", input_tokens),
         ("rmsFirst-", input_tokens // COM_SCALE), ("rmsSecond-", input_tokens // COM_SCALE), ("gate_out-", 11008),
         ("silu_out-", 11008), ("input-", 4096), ("output-", 4096)]
    return [("W", "comW", W), ("R", "comR", R), ("Q", "comQ", Q)]


def pad_rows(t: np.ndarray, n: int) -> np.ndarray:
    """``pad_int`` on the host: rows of n padded with zeros to the next power of two."""
    pad_n = 1 << max(n - 1, 0).bit_length()
    if pad_n == n:
        return t
    rows = t.reshape(-1, n)
    out = np.zeros((rows.shape[0], pad_n), dtype=np.int32)
    out[:, :n] = rows
    return out.reshape(-1)


def commit_tensor(ctx: Context, table: GeneratorTable, tensor: np.ndarray, n: int, max_bits: int = 32) -> np.ndarray:
    """Row commitments of one tensor whose innermost dimension is n (padded to a power of two),
    rows of N*16 scalars (test/commit.cu:63-64)."""
    padded = pad_rows(np.ascontiguousarray(tensor, dtype=np.int32).reshape(-1), n)
    pad_n = 1 << max(n - 1, 0).bit_length()
    wd = pad_n * COM_SCALE
    if padded.size % wd:
        raise ValueError("tensor size is not a multiple of N*16")
    return commit_i32_host(ctx, table, padded, wd, max_bits=max_bits)


def commit_all(ctx: Context, table: GeneratorTable, data_dir, batches: int, lists=None, max_bits: int = 32):
    """Walks data_dir/{W,R,Q}/<name><batch>.bin for batch = batches-1 .. 0, writes data_dir/com*/...
    Missing files are skipped.  Returns {kind: seconds} like the reference's printout."""
    data_dir = Path(data_dir)
    seconds = {}
    for sub, com, files in (lists or file_lists()):
        t_kind = 0.0
        for name, n in files:
            for b in range(batches - 1, -1, -1):
                src = data_dir / sub / f"{name}{b}.bin"
                if not src.exists():
                    continue
                tensor = io.load_int32(src)
                t0 = time.perf_counter()
                rec = commit_tensor(ctx, table, tensor, n, max_bits)
                t_kind += time.perf_counter() - t0
                io.save_blob(data_dir / com / f"{name}{b}.bin", rec)
        seconds[sub] = t_kind
    return seconds
