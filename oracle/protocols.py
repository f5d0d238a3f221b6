"""CPU oracle, part 2: the proving protocols restated on Python integers.

TEST INFRASTRUCTURE ONLY (see ``oracle/bn254.py``).  Field elements are plain integers in
[0, r); tensors are Python lists.  Every function follows the control flow of the reference
function it cites, including its index conventions, so that the recorded round polynomials
("transcript") are the values the reference computes internally and then discards.

Conventions shared by all functions (reference: ``src/ioutils.cu:173-190`` for ``log2ceil``):
multilinear variable 0 is the least-significant index bit; a polynomial is its coefficient
list, lowest degree first (``src/polynomial.cu:26-32``).
"""
from __future__ import annotations

from . import bn254
from .bn254 import R

COM_SCALE = 16  # src/Hyrax.cu:229


def log2ceil(n: int) -> int:
    """The reference's ``Log2``: ceil(log2(n)), and 0 for n in {0, 1}."""
    if n == 0:
        return 0
    n -= 1
    r = 0
    while n > 0:
        n >>= 1
        r += 1
    return r


def inv(x: int) -> int:
    return pow(x, -1, R)


# ----------------------------------------------------------------------------- polynomials
def poly_eq(u: int):
    """eq(u)(t) = (1-u) + (2u-1) t   (src/polynomial.cu:40-45)."""
    return [(1 - u) % R, (2 * u - 1) % R]


def eq2(u: int, v: int) -> int:
    """eq(u, v) = uv + (1-u)(1-v)   (src/polynomial.cu:47-53)."""
    return (2 * u * v - u - v + 1) % R


def poly_mul(a, b):
    out = [0] * (len(a) + len(b) - 1)
    for i, x in enumerate(a):
        for j, y in enumerate(b):
            out[i + j] = (out[i + j] + x * y) % R
    return out


def poly_add(a, b):
    n = max(len(a), len(b))
    return [((a[i] if i < len(a) else 0) + (b[i] if i < len(b) else 0)) % R for i in range(n)]


def poly_scale(a, k):
    return [x * k % R for x in a]


def poly_eval(a, x):
    acc = 0
    for c in reversed(a):
        acc = (acc * x + c) % R
    return acc


def poly_at01(a):
    """p(0) + p(1)."""
    return (a[0] + sum(a)) % R


# ----------------------------------------------------------------------------- folds
def partial_eval(t, ntot, x, c, idx, gap):
    """``FrTensor::partial_eval(N, x, c, id, gap)`` (src/fr-tensor.cu:53-72,168-188,330-344).

    The first ``ntot`` entries are viewed as [other][c][gap]; axis ``c`` is folded with the
    challenges x[idx], x[idx+1], ... pairing neighbours (2j, 2j+1); an odd tail is paired with an
    implicit zero.  Returns the compacted [other][gap] result.
    """
    other = ntot // (c * gap)
    cur = [[t[(o * c + j) * gap:(o * c + j + 1) * gap] for j in range(c)] for o in range(other)]
    cin = c
    for k in range(log2ceil(c)):
        xv = x[idx + k]
        cout = (cin + 1) // 2
        nxt = []
        for o in range(other):
            rows = []
            for j in range(cout):
                lo = cur[o][2 * j]
                if 2 * j + 1 < cin:
                    hi = cur[o][2 * j + 1]
                    rows.append([(a + xv * (b - a)) % R for a, b in zip(lo, hi)])
                else:
                    rows.append([(a - xv * a) % R for a in lo])
            nxt.append(rows)
        cur = nxt
        cin = cout
    out = []
    for o in range(other):
        out.extend(cur[o][0])
    return out


def eq_weights(x, nvars, count):
    """w[j] = prod_k (x[k] if bit k of j else 1-x[k]) for j < count  (closed form of the fold)."""
    w = [1]
    for k in range(nvars):
        xv = x[k]
        w = [a * (1 - xv) % R for a in w] + [a * xv % R for a in w]
    return w[:count]


def tensor_eval(t, u, inner=11008):
    """``FrTensor::operator()(vector<Fr>)`` (src/fr-tensor.cu:346-369).

    A full multilinear evaluation.  When the tensor is smaller than 2^|u| the reference assumes a
    row length of 11008 padded to 16384; ``inner`` carries that constant.
    """
    size = len(t)
    if size < (1 << len(u)):
        t = partial_eval(t, size, u, size // inner, log2ceil(inner), inner)
        t = partial_eval(t, inner, u, inner, 0, 1)
    else:
        t = partial_eval(t, size, u, size, 0, 1)
    return t[0]


# ----------------------------------------------------------------------------- sumcheck kernels
def _split2(A, B, in_size, out_size, v):
    """Two-tensor ``sumcheck_kernel`` (src/prove.cu:29-46): folds A, B in place, returns a, b, c."""
    a = [0] * out_size
    b = [0] * out_size
    c = [0] * out_size
    for g in range(out_size):
        if g + out_size < in_size:
            Aa = (A[g + out_size] - A[g]) % R
            Ba = (B[g + out_size] - B[g]) % R
        else:
            Aa = (-A[g]) % R
            Ba = (-B[g]) % R
        Ab, Bb = A[g], B[g]
        A[g] = (Aa * v + Ab) % R
        B[g] = (Ba * v + Bb) % R
        c[g] = Ab * Bb % R
        b[g] = (Aa * Bb + Ab * Ba) % R
        a[g] = Aa * Ba % R
    return a, b, c


def _split1(X, in_size, out_size, v):
    """One-tensor ``sumcheck_kernel`` (src/prove.cu:14-27)."""
    a = [0] * out_size
    b = [0] * out_size
    for g in range(out_size):
        Xa = (X[g + out_size] - X[g]) % R if g + out_size < in_size else (-X[g]) % R
        Xb = X[g]
        X[g] = (Xa * v + Xb) % R
        b[g] = Xb
        a[g] = Xa
    return a, b


def prove_matmul(A, B, L, N, M, K, u, v, claim):
    """``prove_matmul`` (src/prove.cu:175-210) with its two phases (src/prove.cu:49-117).

    A is [L][N][K], B is [L][M][K] (weights stored [out][in]).  Returns
    ``(A_claim, B_claim, final_claim, transcript)`` where the transcript lists every round
    polynomial.  Raises ``RuntimeError`` where the reference throws.
    """
    A = list(A)
    B = list(B)
    transcript = []
    A = partial_eval(A, len(A), u, N, log2ceil(M), K)
    B = partial_eval(B, len(B), u, M, 0, K)
    u_end = log2ceil(L * N * M)
    v_end = log2ceil(L * K)
    # phase 1: layer variables, most significant first
    size = K * L
    rounds = log2ceil(size // K)
    in_size, out_size = size, size // 2
    eq_acc = 1
    u_l0 = u_end - rounds
    for i in range(rounds):
        v_now = v[v_end - i - 1]
        a, b, c = _split2(A, B, in_size, out_size, v_now)
        a = partial_eval(a, out_size, u[u_l0:], out_size // K, 0, K)
        b = partial_eval(b, out_size, u[u_l0:], out_size // K, 0, K)
        c = partial_eval(c, out_size, u[u_l0:], out_size // K, 0, K)
        p = [sum(c[:K]) % R, sum(b[:K]) % R, sum(a[:K]) % R]
        u_now = u[u_end - i - 1]
        p = poly_mul(p, poly_scale(poly_eq(u_now), eq_acc))
        transcript.append(p)
        if poly_at01(p) != claim % R:
            raise RuntimeError("matmul_phase1: claim != p(0) + p(1)")
        claim = poly_eval(p, v_now)
        in_size, out_size = out_size, out_size // 2
        eq_acc = eq_acc * eq2(u_now, v_now) % R
    # phase 2: inner-product variables, most significant first
    rounds = log2ceil(K)
    in_size = K
    out_size = 1 << (rounds - 1) if rounds else 0
    v_k_end = log2ceil(K)
    for i in range(rounds):
        v_now = v[v_k_end - i - 1]
        a, b, c = _split2(A, B, in_size, out_size, v_now)
        p = [sum(c) * eq_acc % R, sum(b) * eq_acc % R, sum(a) * eq_acc % R]
        transcript.append(p)
        if poly_at01(p) != claim % R:
            raise RuntimeError("matmul_phase2: claim != p(0) + p(1)")
        claim = poly_eval(p, v_now)
        in_size, out_size = out_size, out_size // 2
    if A[0] * B[0] * eq_acc % R != claim:
        raise AssertionError("prove_matmul: final identity failed")
    return A[0], B[0], claim, transcript


def prove_matmul_partial(A, B, L, N, M, K_local, u, v_local):
    """One prover's share of ``prove_matmul`` when the inner dimension is dealt to P = 2^p provers by
    residue class (prover r holds the columns k = k' * P + r).  Not a reference function: the
    reference proves on one GPU.  Because it folds the most significant variable first
    (src/prove.cu:29-46 pairs g with g + out_size), the rounds over the layer variables and over
    the top log2(K) - p inner variables pair elements of the same residue class, so they run on
    each shard alone and the round sums are the sums of the per-shard values returned here.

    ``v_local`` is v without its p lowest entries.  Returns ``(sums, a, b)``: per local round the
    three raw sums (constant, linear, quadratic -- before the eq factors, which are common to all
    shards) and the shard's fully folded values.
    """
    A = partial_eval(list(A), len(A), u, N, log2ceil(M), K_local)
    B = partial_eval(list(B), len(B), u, M, 0, K_local)
    u_end = log2ceil(L * N * M)
    v_end = log2ceil(L * K_local)
    sums = []
    size = K_local * L
    rounds = log2ceil(L)
    in_size, out_size = size, size // 2
    u_l0 = u_end - rounds
    for i in range(rounds):
        a, b, c = _split2(A, B, in_size, out_size, v_local[v_end - i - 1])
        a = partial_eval(a, out_size, u[u_l0:], out_size // K_local, 0, K_local)
        b = partial_eval(b, out_size, u[u_l0:], out_size // K_local, 0, K_local)
        c = partial_eval(c, out_size, u[u_l0:], out_size // K_local, 0, K_local)
        sums.append([sum(c[:K_local]) % R, sum(b[:K_local]) % R, sum(a[:K_local]) % R])
        in_size, out_size = out_size, out_size // 2
    rounds = log2ceil(K_local)
    in_size = K_local
    out_size = 1 << (rounds - 1) if rounds else 0
    for i in range(rounds):
        a, b, c = _split2(A, B, in_size, out_size, v_local[rounds - i - 1])
        sums.append([sum(c) % R, sum(b) % R, sum(a) % R])
        in_size, out_size = out_size, out_size // 2
    return sums, A[0], B[0]


def prove_matmul_finish(parts, L, N, M, K, u, v, claim):
    """Combines the P provers' ``prove_matmul_partial`` results (rank order) into the proof:
    adds the partial sums, runs the last log2(P) rounds over the P folded values, applies the eq
    factors and the reference's round checks.  Returns what ``prove_matmul`` returns."""
    P = len(parts)
    lP, lL, lK = log2ceil(P), log2ceil(L), log2ceil(K)
    assert (1 << lP) == P and K % P == 0
    u_end = log2ceil(L * N * M)
    v_end = log2ceil(L * K)
    local_rounds = lL + lK - lP
    assert all(len(p[0]) == local_rounds for p in parts)
    raw = [[sum(p[0][i][k] for p in parts) % R for k in range(3)] for i in range(local_rounds)]
    A = [p[1] for p in parts]
    B = [p[2] for p in parts]
    in_size, out_size = P, P // 2
    for i in range(lP):
        a, b, c = _split2(A, B, in_size, out_size, v[lP - i - 1])
        raw.append([sum(c) % R, sum(b) % R, sum(a) % R])
        in_size, out_size = out_size, out_size // 2
    transcript = []
    eq_acc = 1
    for i, q in enumerate(raw):
        if i < lL:
            u_now, v_now = u[u_end - i - 1], v[v_end - i - 1]
            p = poly_mul(q, poly_scale(poly_eq(u_now), eq_acc))
        else:
            v_now = v[lK - (i - lL) - 1]
            p = [x * eq_acc % R for x in q]
        transcript.append(p)
        if poly_at01(p) != claim % R:
            raise RuntimeError("prove_matmul (sharded): claim != p(0) + p(1)")
        claim = poly_eval(p, v_now)
        if i < lL:
            eq_acc = eq_acc * eq2(u_now, v_now) % R
    if A[0] * B[0] * eq_acc % R != claim:
        raise AssertionError("prove_matmul (sharded): final identity failed")
    return A[0], B[0], claim, transcript


def reassemble_vectors(first, second, first_size, same_size, last_size):
    """``ReassembleVectors`` (src/ec_operation.cu:74-122): returns the new (first, second)."""
    r1 = second[:same_size] + first[last_size:last_size + first_size] + second[same_size:]
    r2 = second[:same_size] + first[:last_size] + second[same_size:]
    return r1, r2


def prove_elemul(A, B, L, M, N, u, v, claim):
    """``prove_eleMul`` / ``eleMul_sumcheck`` (src/prove.cu:119-172,212-241)."""
    A = list(A)
    B = list(B)
    transcript = []
    first_size = L * M
    size = L * M * N
    if (1 << log2ceil(first_size)) != first_size:
        raise RuntimeError("eleMul_sumcheck: first_size is illegal")
    second_size = size // first_size
    u_end = log2ceil(L * N * M)
    v_end = log2ceil(L * M * N)
    rounds = log2ceil(size)
    in_size, out_size = size, size // 2
    eq_acc = 1
    for i in range(rounds):
        v_now = v[v_end - i - 1]
        a, b, c = _split2(A, B, in_size, out_size, v_now)
        outs = []
        for t in (a, b, c):
            if in_size > second_size:
                t = partial_eval(t, out_size, u[u_end - log2ceil(first_size):],
                                 out_size // second_size, 0, second_size)
                t = partial_eval(t, second_size, u[u_end - log2ceil(size):], second_size, 0, 1)
            else:
                t = partial_eval(t, out_size, u[u_end - log2ceil(size):], out_size, 0, 1)
            outs.append(t[0])
        u_now = u[u_end - i - 1]
        p = poly_mul([outs[2], outs[1], outs[0]], poly_scale(poly_eq(u_now), eq_acc))
        transcript.append(p)
        if poly_at01(p) != claim % R:
            raise RuntimeError("ele_Mul: claim != p(0) + p(1)")
        claim = poly_eval(p, v_now)
        in_size = out_size
        out_size = (1 << (log2ceil(out_size) - 1)) if out_size == second_size else out_size // 2
        eq_acc = eq_acc * eq2(u_now, v_now) % R
    if A[0] * B[0] * eq_acc % R != claim:
        raise AssertionError("prove_eleMul: final identity failed")
    return A[0], B[0], claim, transcript


def combine_claims(X, claims, us, v, size):
    """``combine_claims`` (src/prove.cu:243-301): returns (X~(v), transcript)."""
    assert size == 1 << log2ceil(size)
    X = list(X)
    num = len(claims)
    for uj in us:
        assert len(uj) == len(v)
    assert (1 << len(v)) == size
    claim = sum(claims) % R
    new_u = [list(uj) for uj in us]
    new_v = list(v)
    eq_acc = [1] * num
    in_size, out_size = size, size // 2
    transcript = []
    for _ in range(len(v)):
        v_now = new_v[-1]
        a, b = _split1(X, in_size, out_size, v_now)
        p = [0, 0, 0]
        for j in range(num):
            now_u = new_u[j].pop()
            p1 = [tensor_eval(b, new_u[j]), tensor_eval(a, new_u[j])]
            p1 = poly_mul(p1, poly_eq(now_u))
            p1 = poly_scale(p1, eq_acc[j])
            p = poly_add(p, p1)
            eq_acc[j] = eq_acc[j] * eq2(now_u, v_now) % R
        transcript.append(p)
        if poly_at01(p) != claim:
            raise AssertionError("combine_claims: claim != p(0) + p(1)")
        claim = poly_eval(p, v_now)
        new_v.pop()
        in_size, out_size = out_size, out_size // 2
    ret = X[0]
    if sum(e * ret for e in eq_acc) % R != claim:
        raise AssertionError("combine_claims: final identity failed")
    return ret, transcript


# ----------------------------------------------------------------------------- lookup argument
def _poly_kernel(Ad, Sd, beta, n_out):
    """``tLookup_poly_kernel`` (src/tlookup.cu:64-78)."""
    o0 = [0] * n_out
    o1 = [0] * n_out
    o2 = [0] * n_out
    for t in range(n_out):
        c00 = Ad[t]
        c01 = (Ad[t + n_out] - Ad[t]) % R
        c10 = (Sd[t] + beta) % R
        c11 = (Sd[t + n_out] - Sd[t]) % R
        o0[t] = c00 * c10 % R
        o1[t] = (c01 * c10 + c00 * c11) % R
        o2[t] = c01 * c11 % R
    return o0, o1, o2


def _fold_msb(X, v):
    h = len(X) // 2
    return [(X[g] + v * (X[g + h] - X[g])) % R for g in range(h)]


def _phase1_step(A, S, alpha, beta, C, u):
    """``tLookup_phase1_step_poly`` (src/tlookup.cu:117-151)."""
    if len(A) != len(S):
        raise RuntimeError("A.size != S.size")
    h = len(A) // 2
    t0, t1, t2 = _poly_kernel(A, S, beta, h)
    u_ = u[:-1]
    p0 = [tensor_eval(t0, u_), tensor_eval(t1, u_), tensor_eval(t2, u_)]
    p0 = poly_mul(poly_scale(p0, alpha), poly_eq(u[-1]))
    p1 = [sum(A[:h]) % R, (sum(A[h:2 * h]) - sum(A[:h])) % R]
    return poly_add(poly_add(p0, p1), [C * inv(2) % R])


def _phase2_step(A, S, B, T, m, alpha_, beta, ratio, alpha_sq, u):
    """``tLookup_phase2_step_poly`` (src/tlookup.cu:153-190)."""
    n_out = len(m) // 2
    u_ = u[:-1]
    t0, t1, t2 = _poly_kernel(A, S, beta, n_out)
    p0 = poly_scale([tensor_eval(t0, u_), tensor_eval(t1, u_), tensor_eval(t2, u_)], alpha_)
    coef = ratio * alpha_sq % R
    t0, t1, t2 = _poly_kernel(B, T, beta, n_out)
    p0 = poly_add(p0, poly_scale([tensor_eval(t0, u_), tensor_eval(t1, u_), tensor_eval(t2, u_)], coef))
    p1 = [sum(A[:n_out]) % R, (sum(A[n_out:2 * n_out]) - sum(A[:n_out])) % R]
    t0, t1, t2 = _poly_kernel(m, B, 0, n_out)
    p2 = [sum(t0) % R, sum(t1) % R, sum(t2) % R]
    out = poly_add(poly_mul(poly_eq(u[-1]), p0), p1)
    return poly_add(out, poly_scale(p2, (-ratio) % R))


def lookup_sumcheck(A, S, B, T, m, alpha, beta, C, ratio, u, v1, v2):
    """``tLookup_phase1`` + ``tLookup_phase2`` (src/tlookup.cu:192-244), unrolled from the
    reference's recursion.  Returns (S~(v), final_claim, transcript)."""
    A, S, B, T, m = list(A), list(S), list(B), list(T), list(m)
    u, v1, v2 = list(u), list(v1), list(v2)
    claim = (alpha + alpha * alpha) % R
    alpha_sq = alpha * alpha % R
    transcript = []
    while v1:
        p = _phase1_step(A, S, alpha, beta, C, u)
        transcript.append(p)
        if claim != poly_at01(p):
            raise RuntimeError("tLookup_phase1: claim != p(0) + p(1)")
        vb = v1.pop()
        A = _fold_msb(A, vb)
        S = _fold_msb(S, vb)
        claim = poly_eval(p, vb)
        alpha = alpha * eq2(u[-1], vb) % R
        C = C * inv(2) % R
        u.pop()
    while v2:
        p = _phase2_step(A, S, B, T, m, alpha, beta, ratio, alpha_sq, u)
        transcript.append(p)
        if claim != poly_at01(p):
            raise RuntimeError("tLookup_phase2: claim != p(0) + p(1)")
        vb = v2.pop()
        A, S, B, T, m = (_fold_msb(X, vb) for X in (A, S, B, T, m))
        claim = poly_eval(p, vb)
        e = eq2(u[-1], vb)
        alpha = alpha * e % R
        alpha_sq = alpha_sq * e % R
        u.pop()
    return S[0], claim, transcript


class LookupRange:
    """``tLookupRange`` (src/tlookup.cu:247-343).  ``alpha`` is injected (the reference draws it
    with libff's RNG in the constructor, src/tlookup.cu:247)."""

    def __init__(self, low: int, length: int, alpha: int):
        self.low = low
        self.N = 1 << log2ceil(length)
        self.alpha = alpha % R
        self.beta = self.N % R
        self.T = [(low + i) % R for i in range(self.N)]
        self.B = [inv((t + self.beta) % R) for t in self.T]
        self.m = [0] * self.N

    def table_values(self):
        return self.T

    def prep(self, S):
        """Multiplicities (src/tlookup.cu:265-286): bin index = low 32 bits of (S_i - low)."""
        hist = [0] * self.N
        for s in S:
            hist[((s - self.low) % R) & 0xFFFFFFFF] += 1
        D = len(S)
        if D != 1 << log2ceil(D):
            hist[-self.low] += (1 << log2ceil(D)) - D
        self.m = hist
        return hist

    def padded(self, S, inner=11008, inner_pad=16384, pad_value=0):
        D = len(S)
        Dp = 1 << log2ceil(D)
        if D == Dp:
            return list(S)
        out = []
        for g in range(Dp):
            out.append(S[(g // inner_pad) * inner + g % inner_pad] if g % inner_pad < inner else pad_value)
        return out

    def prove(self, S, v, u, pad_value=0, inner=11008, inner_pad=16384):
        """Returns a dict with the multiplicities, A, the round transcript and the final claims.
        ``u`` holds the ceil(log2 D) field elements the reference draws inside ``prove``
        (src/tlookup.cu:293)."""
        self.prep(S)
        S = self.padded(S, inner, inner_pad, pad_value)
        D = len(S)
        if len(v) != log2ceil(D):
            raise RuntimeError("u.size() != ceilLog2(D)")
        assert len(u) == len(v)
        A = [inv((s + self.beta) % R) for s in S]
        N = self.N
        C = (self.alpha * self.alpha - sum(b * mm for b, mm in zip(self.B, self.m))) % R
        ratio = N * inv(D) % R
        ln = log2ceil(N)
        v1, v2 = v[ln:], v[:ln]
        s_claim, final, tr = lookup_sumcheck(A, S, self.B, self.T, self.m, self.alpha, self.beta,
                                             C, ratio, u, v1, v2)
        return {"m": list(self.m), "A": A, "S_padded": S, "claim": s_claim, "final": final,
                "transcript": tr}


class LookupRangeMapping(LookupRange):
    """``tLookupRangeMapping`` (src/tlookup.cu:350-456): pairs (x, f(x)) folded with a random r."""

    def __init__(self, low: int, length: int, mapped, alpha: int, r: int):
        assert length == 1 << log2ceil(length)
        self.low = low
        self.N = length
        self.alpha = alpha % R
        self.r = r % R
        self.beta = self.N % R
        self.mapped = [x % R for x in mapped]
        self.T = [(low + i + self.mapped[i] * self.r) % R for i in range(self.N)]
        self.B = [inv((t + self.beta) % R) for t in self.T]
        self.m = [0] * self.N

    def prove_pairs(self, S_in, S_out, v, u, inner=11008, inner_pad=16384):
        self.prep(S_in)
        S = [(a + self.r * b) % R for a, b in zip(S_in, S_out)]
        pad_value = self.mapped[-self.low] * self.r % R
        S = self.padded(S, inner, inner_pad, pad_value)
        D = len(S)
        if len(v) != log2ceil(D):
            raise RuntimeError("v.size() != ceilLog2(D)")
        A = [inv((s + self.beta) % R) for s in S]
        N = self.N
        C = (self.alpha * self.alpha - sum(b * mm for b, mm in zip(self.B, self.m))) % R
        ratio = N * inv(D) % R
        ln = log2ceil(N)
        s_claim, final, tr = lookup_sumcheck(A, S, self.B, self.T, self.m, self.alpha, self.beta,
                                             C, ratio, u, v[ln:], v[:ln])
        return {"m": list(self.m), "A": A, "S_padded": S, "claim": s_claim, "final": final,
                "transcript": tr}


# ----------------------------------------------------------------------------- Hyrax
def commit_rows(scalars, wd, gens):
    """Row commitments C_r = sum_i s[r*wd+i] * G_i (src/Hyrax.cu:312-359).  ``scalars`` are signed
    integers or Fr values; the result is a list of normalised affine points."""
    assert len(gens) >= wd and len(scalars) % wd == 0
    return [bn254.msm(scalars[r * wd:(r + 1) * wd], gens[:wd]) for r in range(len(scalars) // wd)]


def hyrax_open(t, e, c, size, N, layer_num, gens, G, d, msm_fn=None):
    """``Hyrax::open`` (src/Hyrax.cu:237-305).  ``d`` is the injected blinding vector of
    16 * 2^ceil(log2 N) field elements (the reference draws it at src/Hyrax.cu:253-256).
    Returns dict(result, z, com_d, com_ad)."""
    if size // N // COM_SCALE < layer_num:
        raise RuntimeError("Size too small: size < N * com_scale * layer_num")
    pad_n = 1 << log2ceil(N)
    new_n = pad_n * COM_SCALE
    assert len(e) == log2ceil(size)
    assert len(d) == new_n
    wd = N * COM_SCALE
    com_d = (msm_fn or bn254.msm)(d, gens[:new_n])
    t = list(t[:size])
    t = partial_eval(t, size, e, (size // layer_num) // wd, log2ceil(wd), wd)
    t = partial_eval(t, wd * layer_num, e, layer_num, log2ceil(size // layer_num), wd)
    x = t[:wd]
    if pad_n != N:
        x = [x[(g // pad_n) * N + g % pad_n] if g % pad_n < N else 0 for g in range(new_n)]
    result = partial_eval(x, new_n, e, new_n, 0, 1)[0]
    z = [(c * xi + di) % R for xi, di in zip(x, d)]
    sum_ad = partial_eval(list(d), new_n, e, new_n, 0, 1)[0]
    com_ad = bn254.scalar_mul(sum_ad, G)
    return {"result": result, "z": z, "com_d": com_d, "com_ad": com_ad}


def host_partial_me(points, begin_vars, add, smul, sub):
    """``host_partial_me<T>`` (include/ec_operation.cuh:37-55) over any group (add/sub/scalar-mul)."""
    pts = list(points)
    for xv in begin_vars:
        out = []
        n = len(pts)
        for i in range((n + 1) // 2):
            if 2 * i + 1 < n:
                out.append(add(pts[2 * i], smul(xv, sub(pts[2 * i + 1], pts[2 * i]))))
            else:
                out.append(sub(pts[2 * i], smul(xv, pts[2 * i])))
        pts = out
    return pts[0]


def hyrax_verify(commitments, proof, e, c, size, N, layer_num, gens, G) -> bool:
    """The two verifier identities of test/HyraxTest.cu:88-125."""
    padd = bn254.add
    psub = lambda a, b: bn254.add(a, bn254.neg(b))
    pmul = bn254.scalar_mul
    wd = N * COM_SCALE
    new_n = (1 << log2ceil(N)) * COM_SCALE
    start_x = log2ceil(wd)
    rows_per_layer = size // wd // layer_num
    layer_c = []
    nrow_vars = len(e) - log2ceil(layer_num) - start_x
    for i in range(layer_num):
        layer_c.append(host_partial_me(commitments[i * rows_per_layer:(i + 1) * rows_per_layer],
                                       e[start_x:start_x + nrow_vars], padd, pmul, psub))
    C_ = host_partial_me(layer_c, e[log2ceil(size // layer_num):], padd, pmul, psub)
    commit_z = bn254.msm(proof["z"], gens[:new_n])
    lhs = padd(pmul(c, C_), proof["com_d"])
    if lhs != commit_z:
        return False
    fadd = lambda a, b: (a + b) % R
    fsub = lambda a, b: (a - b) % R
    fmul = lambda k, a: k * a % R
    az = host_partial_me(proof["z"], e[:start_x], fadd, fmul, fsub)
    left = padd(pmul(c * proof["result"] % R, G), proof["com_ad"])
    return left == pmul(az, G)
