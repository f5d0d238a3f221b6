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


def check_rounds(claim: int, transcript, challenges, max_degree=3) -> int | None:
    """Runs p(0) + p(1) == claim, claim <- p(challenge) over the rounds; returns the final claim or
    None when a round fails, when the number of rounds differs from the number of challenges, or
    when a round polynomial has a non-zero coefficient above its degree bound (`max_degree`: one
    bound for all rounds or one per round; the provers pad every polynomial to four coefficients)."""
    if len(transcript) != len(challenges):
        return None
    bounds = max_degree if isinstance(max_degree, (list, tuple)) else [max_degree] * len(transcript)
    for p, ch, deg in zip(transcript, challenges, bounds):
        if len(p) == 0 or len(p) > 4 or any(c % R for c in p[deg + 1:]):
            return None
        if (p[0] + sum(p)) % R != claim % R:
            return None
        claim = _eval(p, ch)
    return claim


def verify_matmul(claim: int, transcript, u, v, L: int, N: int, M: int, K: int, a_claim: int, b_claim: int) -> bool:
    """Transcript of ``prove_matmul``: layer rounds consume v_L from the top, then inner rounds consume
    v_K from the top; the final claim must equal a_claim * b_claim * prod eq(u_L, v_L)."""
    lL, lK = log2ceil(L), log2ceil(K)
    u_end, v_end = log2ceil(L * N * M), log2ceil(L * K)
    if len(transcript) != lL + lK or len(u) < u_end or len(v) < v_end:
        return False
    chal = [v[v_end - i - 1] for i in range(lL)] + [v[lK - i - 1] for i in range(lK)]
    final = check_rounds(claim, transcript, chal, max_degree=[3] * lL + [2] * lK)
    if final is None:
        return False
    E = 1
    for i in range(lL):
        E = E * _eq2(u[u_end - i - 1], v[v_end - i - 1]) % R
    return a_claim * b_claim * E % R == final


def verify_elemul(claim: int, transcript, u, v, a_claim: int, b_claim: int, size: int | None = None) -> bool:
    """Transcript of ``prove_eleMul``: one round per variable from the top; final claim must equal
    a_claim * b_claim * eq(u, v).  `size` (elements of the tensors, padded per axis as the prover pads
    them) fixes the number of rounds; without it the number of challenges does."""
    n = len(v) if size is None else log2ceil(size)
    if len(transcript) != n or len(u) != n or len(v) != n:
        return False
    chal = [v[n - i - 1] for i in range(n)]
    final = check_rounds(claim, transcript, chal, max_degree=3)
    if final is None:
        return False
    E = 1
    for i in range(n):
        E = E * _eq2(u[i], v[i]) % R
    return a_claim * b_claim * E % R == final


def verify_combine(claims, transcript, us, v, result: int) -> bool:
    """Transcript of ``combine_claims``: final claim must equal result * sum_j eq(u_j, v)."""
    n = len(v)
    if len(transcript) != n or len(us) != len(claims) or any(len(uj) != n for uj in us):
        return False
    final = check_rounds(sum(claims) % R, transcript, [v[n - i - 1] for i in range(n)], max_degree=2)
    if final is None:
        return False
    total = 0
    for uj in us:
        E = 1
        for a, b in zip(uj, v):
            E = E * _eq2(a, b) % R
        total = (total + E) % R
    return result * total % R == final


# ---- lookup argument (LogUp sumcheck of src/tlookup.cu:192-244) ---------------------------------------
def mle_eval(values, point) -> int:
    """Multilinear extension of `values` (length 2^len(point), variable k = bit k of the index) at `point`."""
    vals = [x % R for x in values]
    for xk in point:
        vals = [(vals[2 * i] + xk * (vals[2 * i + 1] - vals[2 * i])) % R for i in range(len(vals) // 2)]
    return vals[0]


def lookup_table_evals(low: int, n: int, beta: int, v_low, mapped=None, r: int = 0):
    """(T~(v_low), B~(v_low)) of the PUBLIC table of a lookup object: T_j = low + j (+ r * mapped_j for a
    mapping table, src/tlookup.cu:16-50), B_j = 1 / (T_j + beta).  O(n) field operations, one batched
    inversion."""
    T = [(low + j + (r * int(mapped[j]) if mapped is not None else 0)) % R for j in range(n)]
    den = [(t + beta) % R for t in T]
    pref, run = [], 1
    for d in den:
        run = run * d % R
        pref.append(run)
    inv = pow(run, -1, R)
    B = [0] * n
    for j in range(n - 1, -1, -1):
        B[j] = inv * (pref[j - 1] if j else 1) % R
        inv = inv * den[j] % R
    return mle_eval(T, v_low), mle_eval(B, v_low)


def verify_lookup(alpha: int, beta: int, n_table: int, d_padded: int, transcript, u, v, finals: dict,
                  table_evals=None) -> bool:
    """Transcript of ``tLookupRange::prove`` / ``tLookupRangeMapping::prove``.

    The argument proves  sum_x [alpha eq(u,x) A(x) (S(x) + beta) + A(x)] + C = alpha + alpha^2  over the
    padded queries, with C = alpha^2 - sum_j B_j m_j restated over the table in the second phase
    (src/tlookup.cu:117-190).  Rounds 0 .. log2(D/N)-1 fold the top variables of A and S, the remaining
    log2 N rounds fold A, S, B, T, m together.  Checks: the number and degree of the round polynomials;
    p(0) + p(1) == claim in every round; and the closing identity at the random point,

        claim_final == a A~ (S~ + beta) + ratio a2 B~ (T~ + beta) + A~ - ratio m~ B~,

    a = alpha prod_all eq(u_i, v_i), a2 = alpha^2 prod_phase2 eq(u_i, v_i), ratio = N / D.
    `finals` holds the claimed A~(v), S~(v), B~, T~, m~ (``Lookup.last_proof``): S~ is what the prover
    returns and the caller ties to an opening of S; A~ and m~ are to be tied to openings of the
    commitments of A and m; `table_evals` = (T~, B~) recomputed from the public table
    (``lookup_table_evals``) replaces trust in the prover's B~ and T~ when given."""
    lD, lN = log2ceil(d_padded), log2ceil(n_table)
    if d_padded != 1 << lD or n_table != 1 << lN or lN > lD:
        return False
    if len(transcript) != lD or len(u) != lD or len(v) != lD:
        return False
    if table_evals is not None and (finals["T"] % R, finals["B"] % R) != (table_evals[0] % R, table_evals[1] % R):
        return False
    n_phase1 = lD - lN
    claim = (alpha + alpha * alpha) % R
    a, a2 = alpha % R, alpha * alpha % R
    for i, p in enumerate(transcript):
        if len(p) == 0 or len(p) > 4:
            return False
        if (p[0] + sum(p)) % R != claim:
            return False
        vb, ub = v[lD - 1 - i], u[lD - 1 - i]
        claim = _eval(p, vb)
        e = _eq2(ub, vb)
        a = a * e % R
        if i >= n_phase1:
            a2 = a2 * e % R
    ratio = n_table * pow(d_padded, -1, R) % R
    A, S, B, T, m = (finals[k] % R for k in ("A", "S", "B", "T", "m"))
    want = (a * A % R * ((S + beta) % R) + ratio * a2 % R * B % R * ((T + beta) % R) + A - ratio * m % R * B) % R
    return want == claim
