"""Verifier for the Hyrax opening and for the sumcheck transcripts the provers emit.

The reference has no verifier (``Hyrax::verify`` is an empty body, src/Hyrax.cu:307-310); its one
external check is the pair of identities in test/HyraxTest.cu:88-125, computed on the host with
libff.  Here the group arithmetic of those identities runs on the GPU (``grape_g1_lincomb``,
``grape_commit_fr``), the field arithmetic of the transcript checks on the host.
"""
from __future__ import annotations

import numpy as np

from . import host
from .host import COM_SCALE, Context, GeneratorTable, commit_fr, decode_field, encode_field

R = host.FR_MODULUS


def log2ceil(n: int) -> int:
    return max(n - 1, 0).bit_length()


def eq_weights(x, count: int):
    """w[j] = prod_k (x_k if bit k of j else 1 - x_k), j < count."""
    w = [1]
    for xv in x:
        w = [a * (1 - xv) % R for a in w] + [a * xv % R for a in w]
    return w[:count]


def lincomb(ctx: Context, points: np.ndarray, scalars) -> bytes:
    """sum_i scalars[i] * points[i] as the 96 bytes of a normalised Jacobian record."""
    pts = np.ascontiguousarray(points, dtype=np.uint32).reshape(-1, 24)
    d_p, d_s, d_o = ctx.upload(pts), ctx.fr_upload(scalars), ctx.alloc(96)
    ctx._check(ctx.lib.grape_g1_lincomb(ctx.handle, d_p.ptr, d_s.ptr, pts.shape[0], d_o.ptr))
    return ctx.download(d_o, 96).tobytes()


def verify_open(ctx: Context, table: GeneratorTable, commitments: np.ndarray, proof, e, c: int, size: int, N: int,
                layer_num: int, G_jacobian: np.ndarray) -> bool:
    """The two identities of test/HyraxTest.cu:88-125:
         c * fold(commitments; row and layer challenges) + com_d == sum_i z_i G_i
         (c * result) * G + com_ad == z~(e[0 .. log2(N*16))) * G
    `commitments`: uint32[layer_num * rows, 24]; `proof`: the object returned by ``hyrax_open``."""
    wd = N * COM_SCALE
    new_n = (1 << log2ceil(N)) * COM_SCALE
    start_x = log2ceil(wd)
    rows = size // wd // layer_num
    com = np.ascontiguousarray(commitments, dtype=np.uint32).reshape(-1, 24)
    if com.shape[0] != rows * layer_num or len(e) != log2ceil(size):
        return False
    w_row = eq_weights(e[start_x:start_x + log2ceil(rows)], rows)
    w_layer = eq_weights(e[log2ceil(size // layer_num):], layer_num)
    weights = [c * wl * wr % R for wl in w_layer for wr in w_row]
    com_d, com_ad = proof.com_raw[0], proof.com_raw[1]
    lhs = lincomb(ctx, np.concatenate([com, com_d.reshape(1, 24)]), weights + [1])
    d_z, d_out = ctx.upload(proof.z_raw), ctx.alloc(96)
    commit_fr(ctx, table, d_z, new_n, new_n, d_out)
    if ctx.download(d_out, 96).tobytes() != lhs:
        return False
    d_e, d_az = ctx.fr_upload(e[:start_x]), ctx.alloc(32)
    ctx.fr_fold(d_z, new_n, d_e, new_n, 1, d_az)
    az = ctx.fr_download(d_az, 1)[0]
    G = np.ascontiguousarray(G_jacobian, dtype=np.uint32).reshape(1, 24)
    left = lincomb(ctx, np.concatenate([G, com_ad.reshape(1, 24)]), [c * proof["result"] % R, 1])
    right = lincomb(ctx, G, [az])
    return left == right


# ---- sumcheck transcripts (host arithmetic) -------------------------------------------------------
def _eval(p, x):
    acc = 0
    for coef in reversed(p):
        acc = (acc * x + coef) % R
    return acc


def _eq2(u, v):
    return (2 * u * v - u - v + 1) % R


def check_rounds(claim: int, transcript, challenges) -> int | None:
    """Runs p(0) + p(1) == claim, claim <- p(challenge) over the rounds; returns the final claim or
    None when a round fails."""
    for p, ch in zip(transcript, challenges):
        if (p[0] + sum(p)) % R != claim % R:
            return None
        claim = _eval(p, ch)
    return claim


def verify_matmul(claim: int, transcript, u, v, L: int, N: int, M: int, K: int, a_claim: int, b_claim: int) -> bool:
    """Transcript of ``prove_matmul``: layer rounds consume v_L from the top, then inner rounds consume
    v_K from the top; the final claim must equal a_claim * b_claim * prod eq(u_L, v_L)."""
    lL, lK = log2ceil(L), log2ceil(K)
    u_end, v_end = log2ceil(L * N * M), log2ceil(L * K)
    if len(transcript) != lL + lK:
        return False
    chal = [v[v_end - i - 1] for i in range(lL)] + [v[lK - i - 1] for i in range(lK)]
    final = check_rounds(claim, transcript, chal)
    if final is None:
        return False
    E = 1
    for i in range(lL):
        E = E * _eq2(u[u_end - i - 1], v[v_end - i - 1]) % R
    return a_claim * b_claim * E % R == final


def verify_elemul(claim: int, transcript, u, v, a_claim: int, b_claim: int) -> bool:
    """Transcript of ``prove_eleMul``: one round per variable from the top; final claim must equal
    a_claim * b_claim * eq(u, v)."""
    n = len(transcript)
    if len(u) < n or len(v) < n:
        return False
    chal = [v[n - i - 1] for i in range(n)]
    final = check_rounds(claim, transcript, chal)
    if final is None:
        return False
    E = 1
    for i in range(n):
        E = E * _eq2(u[i], v[i]) % R
    return a_claim * b_claim * E % R == final


def verify_combine(claims, transcript, us, v, result: int) -> bool:
    """Transcript of ``combine_claims``: final claim must equal result * sum_j eq(u_j, v)."""
    n = len(v)
    if len(transcript) != n:
        return False
    final = check_rounds(sum(claims) % R, transcript, [v[n - i - 1] for i in range(n)])
    if final is None:
        return False
    total = 0
    for uj in us:
        E = 1
        for a, b in zip(uj, v):
            E = E * _eq2(a, b) % R
        total = (total + E) % R
    return result * total % R == final
