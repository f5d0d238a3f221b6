"""The integer arithmetic of the library's field inversion (batched division steps, ``fe_inv`` in
``grape_b200/csrc/field.cuh``), restated word for word on Python integers with every intermediate checked
against the 32- or 64-bit range the kernel holds it in, and the invariants of the method asserted after
every batch: the matrix application is exact, d * a = f and e * a = g modulo m, -2m < d, e < m, and the
loop ends inside the proven bound.  Runs on the CPU; the GPU test of the same routine is
``tests/test_gpu_field.py`` (``grape_diag_field_check``)."""
import random

import pytest

M30 = (1 << 30) - 1
def s32(x):
    x &= 0xffffffff
    return x - (1 << 32) if x >> 31 else x
def chk64(x):
    assert -(1 << 63) <= x < (1 << 63), "int64 overflow"
    return x
def inv_model(a, m, nbits32):
    N = nbits32
    L = (32 * N + 2 + 29) // 30
    MAXB = ((49 * 32 * N + 57) // 17 + 29) // 30 + 1
    m30 = [(m >> (30 * j)) & M30 for j in range(L)]
    m0 = m & 0xffffffff
    x = m0
    for _ in range(5):
        x = (x * ((2 - m0 * x) & 0xffffffff)) & 0xffffffff
    minv30 = x & M30
    assert (minv30 * m) & M30 == 1
    f = m30[:]; g = [(a >> (30 * j)) & M30 for j in range(L)]
    d = [0] * L; e = [0] * L; e[0] = 1
    delta = 1
    batches = 0
    def val(x):
        return sum(v << (30 * j) for j, v in enumerate(x))
    for batch in range(MAXB):
        batches += 1
        f0 = (f[0] | (f[1] << 30)) & 0xffffffff
        g0 = (g[0] | (g[1] << 30)) & 0xffffffff
        u, v, q, r = 1, 0, 0, 1
        left = 30
        while True:
            t = g0 | (1 << left)
            z = (t & -t).bit_length() - 1
            g0 >>= z
            u = (u << z) & 0xffffffff; v = (v << z) & 0xffffffff
            delta += z; left -= z
            if left == 0: break
            if delta > 0:
                delta = -delta
                tf, tu, tv = f0, u, v
                f0 = g0; g0 = (-tf) & 0xffffffff
                u = q; v = r; q = (-tu) & 0xffffffff; r = (-tv) & 0xffffffff
            g0 = (g0 + f0) & 0xffffffff
            q = (q + u) & 0xffffffff; r = (r + v) & 0xffffffff
        su, sv, sq, sr = s32(u), s32(v), s32(q), s32(r)
        F, G = val(f), val(g)
        cf = chk64(su * f[0] + sv * g[0]); cg = chk64(sq * f[0] + sr * g[0])
        assert cf & M30 == 0 and cg & M30 == 0
        cf >>= 30; cg >>= 30
        for j in range(1, L):
            cf = chk64(cf + su * f[j] + sv * g[j]); cg = chk64(cg + sq * f[j] + sr * g[j])
            f[j - 1] = s32(cf) & M30; g[j - 1] = s32(cg) & M30
            cf >>= 30; cg >>= 30
        assert -(1 << 31) <= cf < (1 << 31) and -(1 << 31) <= cg < (1 << 31)
        f[L - 1] = cf; g[L - 1] = cg
        assert val(f) * (1 << 30) == su * F + sv * G and val(g) * (1 << 30) == sq * F + sr * G
        sd = -1 if d[L - 1] < 0 else 0; se = -1 if e[L - 1] < 0 else 0
        md = s32((s32(u) & sd) + (s32(v) & se)); me = s32((s32(q) & sd) + (s32(r) & se))
        Dv, Ev = val(d), val(e)
        cd = chk64(su * d[0] + sv * e[0]); ce = chk64(sq * d[0] + sr * e[0])
        md = s32(md - ((minv30 * (cd & 0xffffffff) + (md & 0xffffffff)) & M30))
        me = s32(me - ((minv30 * (ce & 0xffffffff) + (me & 0xffffffff)) & M30))
        cd = chk64(cd + m30[0] * md); ce = chk64(ce + m30[0] * me)
        assert cd & M30 == 0 and ce & M30 == 0
        cd >>= 30; ce >>= 30
        for j in range(1, L):
            cd = chk64(cd + su * d[j] + sv * e[j] + m30[j] * md); ce = chk64(ce + sq * d[j] + sr * e[j] + m30[j] * me)
            d[j - 1] = s32(cd) & M30; e[j - 1] = s32(ce) & M30
            cd >>= 30; ce >>= 30
        assert -(1 << 31) <= cd < (1 << 31) and -(1 << 31) <= ce < (1 << 31)
        d[L - 1] = cd; e[L - 1] = ce
        assert -2 * m < val(d) < m and -2 * m < val(e) < m, (val(d), val(e))
        assert (val(d) * a - val(f)) % m == 0 and (val(e) * a - val(g)) % m == 0
        if all(x == 0 for x in g): break
    else:
        raise AssertionError("did not finish")
    assert val(f) in (1, -1)
    def carry(x):
        c = 0
        for j in range(L - 1):
            x[j] += c; c = x[j] >> 30; x[j] &= M30
        x[L - 1] += c
    sf = -1 if f[L - 1] < 0 else 0
    d = [(x ^ sf) - sf for x in d]; carry(d)
    for _ in range(2):
        neg = -1 if d[L - 1] < 0 else 0
        d = [x + (m30[j] & neg) for j, x in enumerate(d)]; carry(d)
    t = [x - m30[j] for j, x in enumerate(d)]; carry(t)
    if t[L - 1] >= 0: d = t
    out = val(d)
    assert 0 <= out < m and all(0 <= x <= M30 for x in d)
    # word extraction as in the kernel
    words = []
    for i in range(N):
        bit = 32 * i; j = bit // 30; sh = bit % 30
        w = (d[j] & 0xffffffff) >> sh
        if j + 1 < L: w |= (d[j + 1] & 0xffffffff) << (30 - sh)
        if j + 2 < L: w |= (d[j + 2] & 0xffffffff) << (60 - sh)
        words.append(w & 0xffffffff)
    assert sum(w << (32 * i) for i, w in enumerate(words)) == out
    assert out * a % m == 1
    return out, batches
mods = {
 'bn254_p': (0x30644e72e131a029b85045b68181585d97816a916871ca8d3c208c16d87cfd47, 8),
 'bn254_r': (0x30644e72e131a029b85045b68181585d2833e84879b9709143e1f593f0000001, 8),
 'bls_p': (0x1a0111ea397fe69a4b1ba7b6434bacd764774b84f38512bf6730d2a0f6b0f6241eabfffeb153ffffb9feffffffffaaab, 12),
 'bls_r': (0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001, 8),
}


@pytest.mark.parametrize("name", sorted(mods))
def test_division_step_inverse_model(name):
    m, n = mods[name]
    rng = random.Random(len(name))
    cases = [1, 2, 3, m - 1, m - 2, (m + 1) // 2, 1 << 30, (1 << 30) - 1, m >> 1, 5, 7, 1 << 60]
    cases += [rng.randrange(1, m) for _ in range(300)]
    cases += [rng.randrange(1, 1 << 40) for _ in range(40)] + [m - rng.randrange(1, 1 << 40) for _ in range(40)]
    cases += [1 << k for k in range(0, 32 * n - 2, 7) if (1 << k) < m]
    worst = 0
    for a in cases:
        out, batches = inv_model(a, m, n)
        assert out * a % m == 1
        worst = max(worst, batches)
    assert worst <= ((49 * 32 * n + 57) // 17 + 29) // 30 + 1
