/*
 * CPU oracle, part 3: a plain-C restatement (4 x 64-bit limbs, unsigned __int128) of the
 * reference's commitment and field-tensor algorithms, fast enough to check full-size cases and
 * to serve as the timed host-core baseline.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the product ships links or calls this file; only tests/,
 * the smoke check and the benchmark's CPU-baseline leg load liboracle.so, as the checker / the
 * baseline being reported.
 *
 * Parity status: pinned against oracle/bn254.py (Python big integers) by
 * tests/test_oracle_c.py; the reference itself ships no known-answer vectors.
 *
 * What each function follows (paths inside the reference project):
 *   fe_mul / fe_add / fe_sub          include/field/mont_t.cuh:225-427 (Montgomery residues, R = 2^256)
 *   xyzz_madd / xyzz_add / xyzz_dbl   include/curve/xyzz_t.cuh:129-441 (same group law, EFD formulas)
 *   oracle_table_build                naive_msm, src/ec_operation.cu:15-27: table[w*n + i] = w * G_i, w < 256
 *   oracle_commit_i32                 Hyrax::commit(int*), src/Hyrax.cu:46-87,312-333: four byte windows
 *                                     of |s|, sign by point negation, window sums doubled 8w times
 *   oracle_commit_fr                  Hyrax::commit(FrTensor&), src/Hyrax.cu:128-167,335-359: 32 byte windows
 *   oracle_fr_from_i32                int_to_fr, src/fr-tensor.cu:30-39
 *   oracle_fr_fold                    Fr_partial_me / partial_eval, src/fr-tensor.cu:53-72,168-188,330-344
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef unsigned __int128 u128;
typedef struct { uint64_t w[4]; } fe;

typedef struct {
  uint64_t mod[4], r2[4], one[4], inv;
} field_t;

static const field_t FP = {
    {0x3c208c16d87cfd47ull, 0x97816a916871ca8dull, 0xb85045b68181585dull, 0x30644e72e131a029ull},
    {0xf32cfc5b538afa89ull, 0xb5e71911d44501fbull, 0x47ab1eff0a417ff6ull, 0x06d89f71cab8351full},
    {0xd35d438dc58f0d9dull, 0x0a78eb28f5c70b3dull, 0x666ea36f7879462cull, 0x0e0a77c19a07df2full},
    0x87d20782e4866389ull};
static const field_t FR = {
    {0x43e1f593f0000001ull, 0x2833e84879b97091ull, 0xb85045b68181585dull, 0x30644e72e131a029ull},
    {0x1bb8e645ae216da7ull, 0x53fe3ab1e35c59e3ull, 0x8c49833d53bb8085ull, 0x0216d0b17f4e44a5ull},
    {0xac96341c4ffffffbull, 0x36fc76959f60cd29ull, 0x666ea36f7879462eull, 0x0e0a77c19a07df2full},
    0xc2e1f593efffffffull};

static inline int fe_is_zero(const fe* a) { return (a->w[0] | a->w[1] | a->w[2] | a->w[3]) == 0; }
static inline int fe_eq(const fe* a, const fe* b) { return memcmp(a, b, 32) == 0; }

static inline int geq(const uint64_t* a, const uint64_t* m) {
  for (int i = 3; i >= 0; i--) {
    if (a[i] > m[i]) return 1;
    if (a[i] < m[i]) return 0;
  }
  return 1;
}
static inline void sub_n(uint64_t* r, const uint64_t* a, const uint64_t* b) {
  u128 borrow = 0;
  for (int i = 0; i < 4; i++) {
    u128 d = (u128)a[i] - b[i] - borrow;
    r[i] = (uint64_t)d;
    borrow = (d >> 64) & 1;
  }
}
static inline void fe_add(const field_t* F, fe* r, const fe* a, const fe* b) {
  u128 c = 0;
  fe t;
  for (int i = 0; i < 4; i++) {
    c += (u128)a->w[i] + b->w[i];
    t.w[i] = (uint64_t)c;
    c >>= 64;
  }
  if (geq(t.w, F->mod)) sub_n(t.w, t.w, F->mod);
  *r = t;
}
static inline void fe_neg(const field_t* F, fe* r, const fe* a) {
  if (fe_is_zero(a)) { *r = *a; return; }
  sub_n(r->w, F->mod, a->w);
}
static inline void fe_sub(const field_t* F, fe* r, const fe* a, const fe* b) {
  fe n;
  fe_neg(F, &n, b);
  fe_add(F, r, a, &n);
}
static inline void fe_mul(const field_t* F, fe* r, const fe* a, const fe* b) {
  uint64_t t[6] = {0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 4; i++) {
    u128 c = 0;
    for (int j = 0; j < 4; j++) {
      c += (u128)a->w[j] * b->w[i] + t[j];
      t[j] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[4] = (uint64_t)c;
    t[5] = (uint64_t)(c >> 64);
    uint64_t m = t[0] * F->inv;
    c = (u128)m * F->mod[0] + t[0];
    c >>= 64;
    for (int j = 1; j < 4; j++) {
      c += (u128)m * F->mod[j] + t[j];
      t[j - 1] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[3] = (uint64_t)c;
    t[4] = t[5] + (uint64_t)(c >> 64);
  }
  fe o = {{t[0], t[1], t[2], t[3]}};
  if (t[4] || geq(o.w, F->mod)) sub_n(o.w, o.w, F->mod);
  *r = o;
}
static inline void fe_sqr(const field_t* F, fe* r, const fe* a) { fe_mul(F, r, a, a); }
static void fe_inv(const field_t* F, fe* r, const fe* a) {
  uint64_t e[4] = {F->mod[0] - 2, F->mod[1], F->mod[2], F->mod[3]};
  fe acc;
  memcpy(&acc, F->one, 32);
  for (int i = 3; i >= 0; i--)
    for (int b = 63; b >= 0; b--) {
      fe_sqr(F, &acc, &acc);
      if ((e[i] >> b) & 1) fe_mul(F, &acc, &acc, a);
    }
  *r = acc;
}
static inline void fe_to_mont(const field_t* F, fe* r, const fe* a) {
  fe r2;
  memcpy(&r2, F->r2, 32);
  fe_mul(F, r, a, &r2);
}
static inline void fe_from_mont(const field_t* F, fe* r, const fe* a) {
  fe one = {{1, 0, 0, 0}};
  fe_mul(F, r, a, &one);
}

/* ------------------------------------------------------------------------------------------ */
/* curve: records as in the reference (affine X|Y, (0,0) = infinity; xyzz X|Y|ZZZ|ZZ, ZZ = 0)  */
/* ------------------------------------------------------------------------------------------ */
typedef struct { fe x, y; } affine;
typedef struct { fe x, y, zzz, zz; } xyzz;
typedef struct { fe x, y, z; } jac;

static inline int aff_is_inf(const affine* p) { return fe_is_zero(&p->x) && fe_is_zero(&p->y); }
static inline void xyzz_set_inf(xyzz* p) { memset(p, 0, sizeof(*p)); }
static inline int xyzz_is_inf(const xyzz* p) { return fe_is_zero(&p->zz); }

static void xyzz_dbl(xyzz* r, const xyzz* p) {
  if (xyzz_is_inf(p)) { *r = *p; return; }
  fe U, V, W, S, M, t, X3, Y3;
  fe_add(&FP, &U, &p->y, &p->y);
  fe_sqr(&FP, &V, &U);
  fe_mul(&FP, &W, &U, &V);
  fe_mul(&FP, &S, &p->x, &V);
  fe_sqr(&FP, &t, &p->x);
  fe_add(&FP, &M, &t, &t);
  fe_add(&FP, &M, &M, &t);
  fe_sqr(&FP, &X3, &M);
  fe_sub(&FP, &X3, &X3, &S);
  fe_sub(&FP, &X3, &X3, &S);
  fe_sub(&FP, &t, &S, &X3);
  fe_mul(&FP, &Y3, &M, &t);
  fe_mul(&FP, &t, &W, &p->y);
  fe_sub(&FP, &Y3, &Y3, &t);
  xyzz o;
  o.x = X3;
  o.y = Y3;
  fe_mul(&FP, &o.zz, &V, &p->zz);
  fe_mul(&FP, &o.zzz, &W, &p->zzz);
  *r = o;
}

static void xyzz_add(xyzz* acc, const xyzz* q) {
  if (xyzz_is_inf(q)) return;
  if (xyzz_is_inf(acc)) { *acc = *q; return; }
  fe U1, U2, S1, S2, Pd, Rd, PP, PPP, Q, t, X3, Y3;
  fe_mul(&FP, &U1, &acc->x, &q->zz);
  fe_mul(&FP, &U2, &q->x, &acc->zz);
  fe_mul(&FP, &S1, &acc->y, &q->zzz);
  fe_mul(&FP, &S2, &q->y, &acc->zzz);
  fe_sub(&FP, &Pd, &U2, &U1);
  fe_sub(&FP, &Rd, &S2, &S1);
  if (fe_is_zero(&Pd)) {
    if (fe_is_zero(&Rd)) xyzz_dbl(acc, acc);
    else xyzz_set_inf(acc);
    return;
  }
  fe_sqr(&FP, &PP, &Pd);
  fe_mul(&FP, &PPP, &Pd, &PP);
  fe_mul(&FP, &Q, &U1, &PP);
  fe_sqr(&FP, &X3, &Rd);
  fe_sub(&FP, &X3, &X3, &PPP);
  fe_sub(&FP, &X3, &X3, &Q);
  fe_sub(&FP, &X3, &X3, &Q);
  fe_sub(&FP, &t, &Q, &X3);
  fe_mul(&FP, &Y3, &Rd, &t);
  fe_mul(&FP, &t, &S1, &PPP);
  fe_sub(&FP, &Y3, &Y3, &t);
  acc->x = X3;
  acc->y = Y3;
  fe_mul(&FP, &t, &acc->zz, &q->zz);
  fe_mul(&FP, &acc->zz, &t, &PP);
  fe_mul(&FP, &t, &acc->zzz, &q->zzz);
  fe_mul(&FP, &acc->zzz, &t, &PPP);
}

/* acc += (+/-) q with q affine: 8 multiplications + 2 squarings, as include/curve/xyzz_t.cuh:363-441 */
static void xyzz_madd(xyzz* acc, const affine* q, int negate) {
  if (aff_is_inf(q)) return;
  affine p = *q;
  if (negate) fe_neg(&FP, &p.y, &p.y);
  if (xyzz_is_inf(acc)) {
    acc->x = p.x;
    acc->y = p.y;
    memcpy(&acc->zz, FP.one, 32);
    memcpy(&acc->zzz, FP.one, 32);
    return;
  }
  fe U2, S2, Pd, Rd, PP, PPP, Q, t, X3, Y3;
  fe_mul(&FP, &U2, &p.x, &acc->zz);
  fe_mul(&FP, &S2, &p.y, &acc->zzz);
  fe_sub(&FP, &Pd, &U2, &acc->x);
  fe_sub(&FP, &Rd, &S2, &acc->y);
  if (fe_is_zero(&Pd)) {
    if (fe_is_zero(&Rd)) {
      xyzz d;
      d.x = p.x;
      d.y = p.y;
      memcpy(&d.zz, FP.one, 32);
      memcpy(&d.zzz, FP.one, 32);
      xyzz_dbl(acc, &d);
    } else {
      xyzz_set_inf(acc);
    }
    return;
  }
  fe_sqr(&FP, &PP, &Pd);
  fe_mul(&FP, &PPP, &Pd, &PP);
  fe_mul(&FP, &Q, &acc->x, &PP);
  fe_sqr(&FP, &X3, &Rd);
  fe_sub(&FP, &X3, &X3, &PPP);
  fe_sub(&FP, &X3, &X3, &Q);
  fe_sub(&FP, &X3, &X3, &Q);
  fe_sub(&FP, &t, &Q, &X3);
  fe_mul(&FP, &Y3, &Rd, &t);
  fe_mul(&FP, &t, &acc->y, &PPP);
  fe_sub(&FP, &Y3, &Y3, &t);
  acc->x = X3;
  acc->y = Y3;
  fe_mul(&FP, &acc->zz, &acc->zz, &PP);
  fe_mul(&FP, &acc->zzz, &acc->zzz, &PPP);
}

static void xyzz_to_affine(affine* r, const xyzz* p) {
  if (xyzz_is_inf(p)) { memset(r, 0, sizeof(*r)); return; }
  fe t, izz, izzz;
  fe_mul(&FP, &t, &p->zz, &p->zzz);
  fe_inv(&FP, &t, &t);
  fe_mul(&FP, &izz, &t, &p->zzz);
  fe_mul(&FP, &izzz, &t, &p->zz);
  fe_mul(&FP, &r->x, &p->x, &izz);
  fe_mul(&FP, &r->y, &p->y, &izzz);
}

static void jac_store_normalised(jac* out, const xyzz* p) {
  if (xyzz_is_inf(p)) {
    memcpy(&out->x, FP.one, 32);
    memcpy(&out->y, FP.one, 32);
    memset(&out->z, 0, 32);
    return;
  }
  affine a;
  xyzz_to_affine(&a, p);
  out->x = a.x;
  out->y = a.y;
  memcpy(&out->z, FP.one, 32);
}

static void xyzz_from_jac(xyzz* r, const jac* j) {
  if (fe_is_zero(&j->z)) { xyzz_set_inf(r); return; }
  r->x = j->x;
  r->y = j->y;
  fe_sqr(&FP, &r->zz, &j->z);
  fe_mul(&FP, &r->zzz, &r->zz, &j->z);
}

/* ------------------------------------------------------------------------------------------ */
/* exported API (ctypes)                                                                       */
/* ------------------------------------------------------------------------------------------ */
int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* field element-wise: op 0 add, 1 sub, 2 mul; field 0 = Fr, 1 = Fp */
void oracle_fe_binary(int field, int op, const fe* a, const fe* b, fe* out, uint64_t n) {
  const field_t* F = field ? &FP : &FR;
#pragma omp parallel for
  for (int64_t i = 0; i < (int64_t)n; i++) {
    if (op == 0) fe_add(F, &out[i], &a[i], &b[i]);
    else if (op == 1) fe_sub(F, &out[i], &a[i], &b[i]);
    else fe_mul(F, &out[i], &a[i], &b[i]);
  }
}

void oracle_fr_from_i32(const int32_t* in, fe* out, uint64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < (int64_t)n; i++) {
    int64_t v = in[i];
    fe t = {{(uint64_t)(v < 0 ? -v : v), 0, 0, 0}};
    fe_to_mont(&FR, &t, &t);
    if (v < 0) fe_neg(&FR, &t, &t);
    out[i] = t;
  }
}

/* table[w * n + i] = w * G_i for w < 256 (row 0 = infinity), affine.  The 255 multiples of one
 * generator are normalised together (one inversion per generator). */
void oracle_table_build(const jac* gens, uint64_t n, affine* table) {
#pragma omp parallel for
  for (int64_t i = 0; i < (int64_t)n; i++) {
    xyzz g, acc, pts[256];
    fe pref[256], run, inv, zp, t;
    xyzz_from_jac(&g, &gens[i]);
    xyzz_set_inf(&acc);
    memcpy(&run, FP.one, 32);
    for (int w = 0; w < 256; w++) {
      pts[w] = acc;
      if (!xyzz_is_inf(&acc)) {
        fe_mul(&FP, &zp, &acc.zz, &acc.zzz);
        fe_mul(&FP, &run, &run, &zp);
      }
      pref[w] = run;
      xyzz_add(&acc, &g);
    }
    fe_inv(&FP, &inv, &run);
    for (int w = 255; w >= 0; w--) {
      affine* out = &table[(uint64_t)w * n + i];
      if (xyzz_is_inf(&pts[w])) { memset(out, 0, sizeof(*out)); continue; }
      fe zinv;
      if (w == 0) zinv = inv; else fe_mul(&FP, &zinv, &inv, &pref[w - 1]);
      fe_mul(&FP, &zp, &pts[w].zz, &pts[w].zzz);
      fe_mul(&FP, &inv, &inv, &zp);
      fe_mul(&FP, &t, &zinv, &pts[w].zzz);
      fe_mul(&FP, &out->x, &pts[w].x, &t);
      fe_mul(&FP, &t, &zinv, &pts[w].zz);
      fe_mul(&FP, &out->y, &pts[w].y, &t);
    }
  }
}

/* one commitment row with byte windows: scalars given as nbytes little-endian magnitude bytes */
static void commit_row_bytes(const uint8_t* mags, const uint8_t* negs, int nbytes, uint64_t wd,
                             const affine* table, uint64_t npoints, jac* out) {
  xyzz total;
  xyzz_set_inf(&total);
  for (int w = nbytes - 1; w >= 0; w--) {
    for (int k = 0; k < 8; k++) xyzz_dbl(&total, &total);
    xyzz sum;
    xyzz_set_inf(&sum);
    for (uint64_t i = 0; i < wd; i++) {
      uint8_t d = mags[i * nbytes + w];
      if (d) xyzz_madd(&sum, &table[(uint64_t)d * npoints + i], negs ? negs[i] : 0);
    }
    xyzz_add(&total, &sum);
  }
  jac_store_normalised(out, &total);
}

/* C_r = sum_i s[r*wd + i] * G_i; rows [row_begin, row_end) only (for bounded samples) */
void oracle_commit_i32(const int32_t* scalars, uint64_t wd, uint64_t row_begin, uint64_t row_end,
                       const affine* table, uint64_t npoints, jac* out) {
#pragma omp parallel
  {
    uint8_t* mags = (uint8_t*)malloc(wd * 4);
    uint8_t* negs = (uint8_t*)malloc(wd);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = (int64_t)row_begin; r < (int64_t)row_end; r++) {
      for (uint64_t i = 0; i < wd; i++) {
        int64_t v = scalars[(uint64_t)r * wd + i];
        uint32_t a = (uint32_t)(v < 0 ? -v : v);
        negs[i] = v < 0;
        memcpy(&mags[i * 4], &a, 4);
      }
      commit_row_bytes(mags, negs, 4, wd, table, npoints, &out[r - row_begin]);
    }
    free(mags);
    free(negs);
  }
}

void oracle_commit_fr(const fe* scalars, uint64_t wd, uint64_t row_begin, uint64_t row_end,
                      const affine* table, uint64_t npoints, jac* out) {
#pragma omp parallel
  {
    uint8_t* mags = (uint8_t*)malloc(wd * 32);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = (int64_t)row_begin; r < (int64_t)row_end; r++) {
      for (uint64_t i = 0; i < wd; i++) {
        fe s;
        fe_from_mont(&FR, &s, &scalars[(uint64_t)r * wd + i]);
        memcpy(&mags[i * 32], &s, 32);
      }
      commit_row_bytes(mags, NULL, 32, wd, table, npoints, &out[r - row_begin]);
    }
    free(mags);
  }
}

/* In-place fold exactly as the reference does it: view [other][c][gap], log2ceil(c) passes pairing
 * (2j, 2j+1) with challenge x[id + pass], then compaction to [other][gap]. */
void oracle_fr_fold(fe* t, uint64_t ntot, const fe* x, uint32_t c, uint32_t id, uint64_t gap) {
  uint64_t other = ntot / ((uint64_t)c * gap);
  uint64_t dim = (uint64_t)c * gap;
  uint32_t cin = c;
  uint64_t g = gap;
  uint32_t passes = 0;
  for (uint32_t v = c - 1; c > 1 && v > 0; v >>= 1) passes++;
  for (uint32_t p = 0; p < passes; p++) {
    uint32_t cout = (cin + 1) / 2;
    const fe* xv = &x[id + p];
#pragma omp parallel for collapse(2)
    for (int64_t o = 0; o < (int64_t)other; o++)
      for (int64_t j = 0; j < (int64_t)cout; j++)
        for (uint64_t k = 0; k < gap; k++) {
          fe* lo = &t[o * dim + (2 * j) * g + k];
          fe d, m;
          if ((uint32_t)(2 * j + 1) < cin) {
            fe* hi = &t[o * dim + (2 * j + 1) * g + k];
            fe_sub(&FR, &d, hi, lo);
            fe_mul(&FR, &m, xv, &d);
            fe_add(&FR, lo, lo, &m);
          } else {
            fe_mul(&FR, &m, xv, lo);
            fe_sub(&FR, lo, lo, &m);
          }
        }
    g <<= 1;
    cin = cout;
  }
  for (uint64_t o = 1; o < other; o++) memmove(&t[o * gap], &t[o * dim], gap * sizeof(fe));
}

/* prove_matmul (src/prove.cu:175-210 with matmul_sumcheck_phase2, :85-117) for one layer (L = 1):
 * A is [N][K], B is [M][K], both int32.  u and v are the challenge vectors, *claim the claimed value of
 * the product's multilinear extension at u.  Writes the two final claims, the claim after the last
 * round, and three coefficients per round.  Returns 0, or 1 + the index of the first round whose
 * check p(0) + p(1) == claim fails (the reference throws there), or -1 when A*B*eq != claim at the end. */
static uint32_t log2ceil_u32(uint64_t n) {
  uint32_t r = 0;
  if (n == 0) return 0;
  n--;
  while (n) { n >>= 1; r++; }
  return r;
}

int oracle_prove_matmul_l1(const int32_t* A, const int32_t* B, uint32_t N, uint32_t M, uint32_t K, const fe* u,
                           const fe* v, fe* claim, fe* out_a, fe* out_b, fe* transcript) {
  fe* a = (fe*)malloc((size_t)N * K * sizeof(fe));
  fe* b = (fe*)malloc((size_t)M * K * sizeof(fe));
  if (!a || !b) { free(a); free(b); return -2; }
  oracle_fr_from_i32(A, a, (uint64_t)N * K);
  oracle_fr_from_i32(B, b, (uint64_t)M * K);
  oracle_fr_fold(a, (uint64_t)N * K, u, N, log2ceil_u32(M), K);
  oracle_fr_fold(b, (uint64_t)M * K, u, M, 0, K);
  const uint32_t rounds = log2ceil_u32(K);
  uint64_t in_size = K, out_size = rounds ? ((uint64_t)1 << (rounds - 1)) : 0;
  int rc = 0;
  const int nt = oracle_threads();
  fe* part = (fe*)calloc((size_t)nt * 3, sizeof(fe));
  for (uint32_t i = 0; i < rounds && rc == 0; i++) {
    const fe* vn = &v[rounds - i - 1];
    memset(part, 0, (size_t)nt * 3 * sizeof(fe));
#pragma omp parallel num_threads(nt)
    {
      int tid = 0;
#ifdef _OPENMP
      tid = omp_get_thread_num();
#endif
      fe s0, s1, s2;
      memset(&s0, 0, sizeof s0);
      memset(&s1, 0, sizeof s1);
      memset(&s2, 0, sizeof s2);
#pragma omp for
      for (int64_t g = 0; g < (int64_t)out_size; g++) {
        fe Aa, Ba, Ab = a[g], Bb = b[g], t0, t1;
        if ((uint64_t)g + out_size < in_size) {
          fe_sub(&FR, &Aa, &a[g + out_size], &Ab);
          fe_sub(&FR, &Ba, &b[g + out_size], &Bb);
        } else {
          fe_neg(&FR, &Aa, &Ab);
          fe_neg(&FR, &Ba, &Bb);
        }
        fe_mul(&FR, &t0, &Aa, vn);
        fe_add(&FR, &a[g], &t0, &Ab);
        fe_mul(&FR, &t0, &Ba, vn);
        fe_add(&FR, &b[g], &t0, &Bb);
        fe_mul(&FR, &t0, &Ab, &Bb);
        fe_add(&FR, &s0, &s0, &t0);
        fe_mul(&FR, &t0, &Aa, &Bb);
        fe_mul(&FR, &t1, &Ab, &Ba);
        fe_add(&FR, &t0, &t0, &t1);
        fe_add(&FR, &s1, &s1, &t0);
        fe_mul(&FR, &t0, &Aa, &Ba);
        fe_add(&FR, &s2, &s2, &t0);
      }
      part[3 * tid] = s0;
      part[3 * tid + 1] = s1;
      part[3 * tid + 2] = s2;
    }
    fe p[3];
    memset(p, 0, sizeof p);
    for (int t = 0; t < nt; t++)
      for (int k = 0; k < 3; k++) fe_add(&FR, &p[k], &p[k], &part[3 * t + k]);
    for (int k = 0; k < 3; k++) transcript[3 * i + k] = p[k];
    fe s, t2;
    fe_add(&FR, &s, &p[0], &p[0]);   /* p(0) + p(1) = 2 c0 + c1 + c2 */
    fe_add(&FR, &s, &s, &p[1]);
    fe_add(&FR, &s, &s, &p[2]);
    if (!fe_eq(&s, claim)) { rc = 1 + (int)i; break; }
    fe_mul(&FR, &t2, &p[2], vn);     /* claim = (c2 v + c1) v + c0 */
    fe_add(&FR, &t2, &t2, &p[1]);
    fe_mul(&FR, &t2, &t2, vn);
    fe_add(&FR, claim, &t2, &p[0]);
    in_size = out_size;
    out_size /= 2;
  }
  if (rc == 0) {
    fe prod;
    fe_mul(&FR, &prod, &a[0], &b[0]);
    if (!fe_eq(&prod, claim)) rc = -1;
    *out_a = a[0];
    *out_b = b[0];
  }
  free(part);
  free(a);
  free(b);
  return rc;
}

/* ------------------------------------------------------------------------------------------ */
/* tLookupRange::prove (src/tlookup.cu:288-343 with tLookup_phase1 / phase2, :192-244, and the     */
/* step polynomials, :117-190) for a power-of-two number of int32 queries.                         */
/* ------------------------------------------------------------------------------------------ */
static void fr_set_u64(fe* r, uint64_t v) {
  fe t;
  memset(&t, 0, sizeof t);
  t.w[0] = v;
  fe_to_mont(&FR, r, &t);
}
static void fr_set_i64(fe* r, int64_t v) {
  if (v >= 0) {
    fr_set_u64(r, (uint64_t)v);
  } else {
    fe t;
    fr_set_u64(&t, (uint64_t)(-v));
    fe_neg(&FR, r, &t);
  }
}
/* sum of n elements (parallel) */
static void fr_sum(fe* out, const fe* x, uint64_t n) {
  const int nt = oracle_threads();
  fe* part = (fe*)calloc((size_t)nt, sizeof(fe));
#pragma omp parallel num_threads(nt)
  {
    int tid = 0;
#ifdef _OPENMP
    tid = omp_get_thread_num();
#endif
    fe acc;
    memset(&acc, 0, sizeof acc);
#pragma omp for
    for (int64_t i = 0; i < (int64_t)n; i++) fe_add(&FR, &acc, &acc, &x[i]);
    part[tid] = acc;
  }
  memset(out, 0, sizeof *out);
  for (int t = 0; t < nt; t++) fe_add(&FR, out, out, &part[t]);
  free(part);
}
/* multilinear evaluation of t[0..2^nv) at u[0..nv), lowest variable first, destroying t
 * (FrTensor::operator()(vector<Fr>), src/fr-tensor.cu:346-369) */
static void mle_eval(fe* out, fe* t, uint32_t nv, const fe* u, fe* tmp) {
  uint64_t n = (uint64_t)1 << nv;
  fe* src = t;
  fe* dst = tmp;   /* ping-pong: a pass never writes the buffer it reads (tmp holds 2^(nv-1) elements) */
  for (uint32_t k = 0; k < nv; k++) {
    const uint64_t h = n / 2;
#pragma omp parallel for if (h > 4096)
    for (int64_t j = 0; j < (int64_t)h; j++) {
      fe d, m;
      fe_sub(&FR, &d, &src[2 * j + 1], &src[2 * j]);
      fe_mul(&FR, &m, &u[k], &d);
      fe_add(&FR, &dst[j], &src[2 * j], &m);
    }
    fe* sw = src;
    src = dst;
    dst = sw;
    n = h;
  }
  *out = src[0];
}
/* tLookup_poly_kernel (src/tlookup.cu:64-78) followed by the three evaluations at u_: p[k] = t_k~(u_) */
static void poly_terms_eval(fe p[3], const fe* X, const fe* Y, const fe* shift, uint64_t h, uint32_t nv, const fe* u,
                            fe* t0, fe* t1, fe* t2, fe* tmp) {
#pragma omp parallel for if (h > 4096)
  for (int64_t t = 0; t < (int64_t)h; t++) {
    fe c01, c10, c11, a, b;
    fe_sub(&FR, &c01, &X[t + h], &X[t]);
    fe_add(&FR, &c10, &Y[t], shift);
    fe_sub(&FR, &c11, &Y[t + h], &Y[t]);
    fe_mul(&FR, &t0[t], &X[t], &c10);
    fe_mul(&FR, &a, &c01, &c10);
    fe_mul(&FR, &b, &X[t], &c11);
    fe_add(&FR, &t1[t], &a, &b);
    fe_mul(&FR, &t2[t], &c01, &c11);
  }
  if (u) {
    mle_eval(&p[0], t0, nv, u, tmp);
    mle_eval(&p[1], t1, nv, u, tmp);
    mle_eval(&p[2], t2, nv, u, tmp);
  } else {
    fr_sum(&p[0], t0, h);
    fr_sum(&p[1], t1, h);
    fr_sum(&p[2], t2, h);
  }
}
static void fold_msb(fe* X, uint64_t h, const fe* v) {
#pragma omp parallel for if (h > 4096)
  for (int64_t g = 0; g < (int64_t)h; g++) {
    fe d, m;
    fe_sub(&FR, &d, &X[g + h], &X[g]);
    fe_mul(&FR, &m, v, &d);
    fe_add(&FR, &X[g], &X[g], &m);
  }
}
static void poly_eval4(fe* out, const fe p[4], const fe* x) {
  fe acc = p[3];
  for (int k = 2; k >= 0; k--) {
    fe_mul(&FR, &acc, &acc, x);
    fe_add(&FR, &acc, &acc, &p[k]);
  }
  *out = acc;
}
static void eq2_fr(fe* out, const fe* u, const fe* v, const fe* one) {  /* uv + (1-u)(1-v) */
  fe uv, a, b;
  fe_mul(&FR, &uv, u, v);
  fe_sub(&FR, &a, one, u);
  fe_sub(&FR, &b, one, v);
  fe_mul(&FR, &a, &a, &b);
  fe_add(&FR, out, &uv, &a);
}

/* q: D = 2^lD int32 queries in [low, low + N), N = 2^lN <= D.  alpha: the lookup's random scalar, u, v:
 * lD challenges each (u is what the reference draws inside prove).  Outputs: multiplicities m_out[N],
 * S~(v), the claim after the last round, four coefficients per round.  Returns 0, 1 + round index
 * of a failed check, or -3 when a query lies outside the table. */
int oracle_lookup_range(const int32_t* q, uint32_t lD, int32_t low, uint32_t lN, const fe* alpha_in, const fe* u_in,
                        const fe* v, uint32_t* m_out, fe* s_claim, fe* final_claim, fe* transcript) {
  const uint64_t D = (uint64_t)1 << lD, N = (uint64_t)1 << lN;
  fe one, beta, alpha = *alpha_in, alpha_sq, C, ratio, two_inv, claim;
  fr_set_u64(&one, 1);
  fr_set_u64(&beta, N);
  memset(m_out, 0, N * sizeof(uint32_t));
  for (uint64_t i = 0; i < D; i++) {
    int64_t k = (int64_t)q[i] - low;
    if (k < 0 || (uint64_t)k >= N) return -3;
    m_out[k]++;
  }
  fe* T = (fe*)malloc(N * sizeof(fe));
  fe* B = (fe*)malloc(N * sizeof(fe));
  fe* Mf = (fe*)malloc(N * sizeof(fe));
  fe* S = (fe*)malloc(D * sizeof(fe));
  fe* A = (fe*)malloc(D * sizeof(fe));
  fe* t0 = (fe*)malloc(D / 2 * sizeof(fe));
  fe* t1 = (fe*)malloc(D / 2 * sizeof(fe));
  fe* t2 = (fe*)malloc(D / 2 * sizeof(fe));
  fe* u = (fe*)malloc((lD + 1) * sizeof(fe));
  fe* tmp = (fe*)malloc((D / 4 + 1) * sizeof(fe));
  memcpy(u, u_in, lD * sizeof(fe));
#pragma omp parallel for
  for (int64_t t = 0; t < (int64_t)N; t++) {
    fe s;
    fr_set_i64(&T[t], (int64_t)low + t);
    fe_add(&FR, &s, &T[t], &beta);
    fe_inv(&FR, &B[t], &s);
    fr_set_u64(&Mf[t], m_out[t]);
  }
  oracle_fr_from_i32(q, S, D);
#pragma omp parallel for
  for (int64_t i = 0; i < (int64_t)D; i++) A[i] = B[(int64_t)q[i] - low];   /* = 1 / (S_i + beta) */
  /* C = alpha^2 - sum B m;  ratio = N / D;  claim = alpha + alpha^2 */
  fe_mul(&FR, &alpha_sq, &alpha, &alpha);
  {
    fe acc, prod;
    memset(&acc, 0, sizeof acc);
    for (uint64_t t = 0; t < N; t++) {
      fe_mul(&FR, &prod, &B[t], &Mf[t]);
      fe_add(&FR, &acc, &acc, &prod);
    }
    fe_sub(&FR, &C, &alpha_sq, &acc);
    fe dfe, dinv, nfe;
    fr_set_u64(&dfe, D);
    fr_set_u64(&nfe, N);
    fe_inv(&FR, &dinv, &dfe);
    fe_mul(&FR, &ratio, &nfe, &dinv);
    fe two;
    fr_set_u64(&two, 2);
    fe_inv(&FR, &two_inv, &two);
  }
  fe_add(&FR, &claim, &alpha, &alpha_sq);
  int rc = 0;
  uint32_t nu = lD, round = 0;
  uint64_t n = D;
  /* phase 1: the variables beyond the table's, last challenge first */
  for (uint32_t i = 0; i < lD - lN && rc == 0; i++, round++) {
    const uint64_t h = n / 2;
    const fe* ul = &u[nu - 1];
    const fe* vb = &v[lD - 1 - i];
    fe p0[3], p[4], e0, e1, sl, sh, half_c;
    poly_terms_eval(p0, A, S, &beta, h, nu - 1, u, t0, t1, t2, tmp);
    for (int k = 0; k < 3; k++) fe_mul(&FR, &p0[k], &p0[k], &alpha);
    fe_sub(&FR, &e0, &one, ul);            /* eq(u)(t) = (1-u) + (2u-1) t */
    fe_add(&FR, &e1, ul, ul);
    fe_sub(&FR, &e1, &e1, &one);
    fe a, b;
    fe_mul(&FR, &p[0], &p0[0], &e0);
    fe_mul(&FR, &a, &p0[1], &e0);
    fe_mul(&FR, &b, &p0[0], &e1);
    fe_add(&FR, &p[1], &a, &b);
    fe_mul(&FR, &a, &p0[2], &e0);
    fe_mul(&FR, &b, &p0[1], &e1);
    fe_add(&FR, &p[2], &a, &b);
    fe_mul(&FR, &p[3], &p0[2], &e1);
    fr_sum(&sl, A, h);
    fr_sum(&sh, A + h, h);
    fe_add(&FR, &p[0], &p[0], &sl);
    fe_sub(&FR, &sh, &sh, &sl);
    fe_add(&FR, &p[1], &p[1], &sh);
    fe_mul(&FR, &half_c, &C, &two_inv);
    fe_add(&FR, &p[0], &p[0], &half_c);
    for (int k = 0; k < 4; k++) transcript[4 * round + k] = p[k];
    fe s01 = p[0];
    for (int k = 0; k < 4; k++) fe_add(&FR, &s01, &s01, &p[k]);
    if (!fe_eq(&s01, &claim)) { rc = 1 + (int)round; break; }
    fold_msb(A, h, vb);
    fold_msb(S, h, vb);
    poly_eval4(&claim, p, vb);
    fe e;
    eq2_fr(&e, ul, vb, &one);
    fe_mul(&FR, &alpha, &alpha, &e);
    C = half_c;
    nu--;
    n = h;
  }
  /* phase 2: the table's variables */
  uint64_t nt = N;
  for (uint32_t i = 0; i < lN && rc == 0; i++, round++) {
    const uint64_t h = nt / 2;
    const fe* ul = &u[nu - 1];
    const fe* vb = &v[lN - 1 - i];
    fe pa[3], pb[3], pm[3], p0[3], p[4], e0, e1, coef, sl, sh, zero, nratio;
    memset(&zero, 0, sizeof zero);
    poly_terms_eval(pa, A, S, &beta, h, nu - 1, u, t0, t1, t2, tmp);
    poly_terms_eval(pb, B, T, &beta, h, nu - 1, u, t0, t1, t2, tmp);
    poly_terms_eval(pm, Mf, B, &zero, h, 0, NULL, t0, t1, t2, tmp);
    fe_mul(&FR, &coef, &ratio, &alpha_sq);
    for (int k = 0; k < 3; k++) {
      fe x, y;
      fe_mul(&FR, &x, &pa[k], &alpha);
      fe_mul(&FR, &y, &pb[k], &coef);
      fe_add(&FR, &p0[k], &x, &y);
    }
    fe_sub(&FR, &e0, &one, ul);
    fe_add(&FR, &e1, ul, ul);
    fe_sub(&FR, &e1, &e1, &one);
    fe a, b;
    fe_mul(&FR, &p[0], &p0[0], &e0);
    fe_mul(&FR, &a, &p0[1], &e0);
    fe_mul(&FR, &b, &p0[0], &e1);
    fe_add(&FR, &p[1], &a, &b);
    fe_mul(&FR, &a, &p0[2], &e0);
    fe_mul(&FR, &b, &p0[1], &e1);
    fe_add(&FR, &p[2], &a, &b);
    fe_mul(&FR, &p[3], &p0[2], &e1);
    fr_sum(&sl, A, h);
    fr_sum(&sh, A + h, h);
    fe_add(&FR, &p[0], &p[0], &sl);
    fe_sub(&FR, &sh, &sh, &sl);
    fe_add(&FR, &p[1], &p[1], &sh);
    fe_neg(&FR, &nratio, &ratio);
    for (int k = 0; k < 3; k++) {
      fe x;
      fe_mul(&FR, &x, &pm[k], &nratio);
      fe_add(&FR, &p[k], &p[k], &x);
    }
    for (int k = 0; k < 4; k++) transcript[4 * round + k] = p[k];
    fe s01 = p[0];
    for (int k = 0; k < 4; k++) fe_add(&FR, &s01, &s01, &p[k]);
    if (!fe_eq(&s01, &claim)) { rc = 1 + (int)round; break; }
    fold_msb(A, h, vb);
    fold_msb(S, h, vb);
    fold_msb(B, h, vb);
    fold_msb(T, h, vb);
    fold_msb(Mf, h, vb);
    poly_eval4(&claim, p, vb);
    fe e;
    eq2_fr(&e, ul, vb, &one);
    fe_mul(&FR, &alpha, &alpha, &e);
    fe_mul(&FR, &alpha_sq, &alpha_sq, &e);
    nu--;
    nt = h;
  }
  *s_claim = S[0];
  *final_claim = claim;
  free(T); free(B); free(Mf); free(S); free(A); free(t0); free(t1); free(t2); free(u); free(tmp);
  return rc;
}

/* ------------------------------------------------------------------------------------------ */
/* Host scalar / group operations and the seeded random stream, exported for the libff stand-in */
/* that lets the reference's own sources compile (oracle/ref_shim).                              */
/* ------------------------------------------------------------------------------------------ */
void oracle_fr_add(const fe* a, const fe* b, fe* out) { fe_add(&FR, out, a, b); }
void oracle_fr_sub(const fe* a, const fe* b, fe* out) { fe_sub(&FR, out, a, b); }
void oracle_fr_mul(const fe* a, const fe* b, fe* out) { fe_mul(&FR, out, a, b); }
void oracle_fr_inv(const fe* a, fe* out) { fe_inv(&FR, out, a); }
void oracle_fr_from_i64(int64_t v, fe* out) {
  uint64_t mag = v < 0 ? (uint64_t)(-(v + 1)) + 1 : (uint64_t)v;
  fe t = {{mag, 0, 0, 0}};
  fe_to_mont(&FR, &t, &t);
  if (v < 0) fe_neg(&FR, &t, &t);
  *out = t;
}

/* SplitMix64; one draw = eight outputs (lo words, then hi words), value (lo + hi * 2^256) mod r */
static uint64_t splitmix_next(uint64_t* state) {
  *state += 0x9E3779B97F4A7C15ull;
  uint64_t z = *state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
uint64_t oracle_rng_init(uint64_t seed, uint64_t tag) {
  return seed * 0x9E3779B97F4A7C15ull + tag * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
}
void oracle_rng_fr(uint64_t* state, fe* out) {
  fe lo, hi, r2;
  for (int i = 0; i < 4; i++) lo.w[i] = splitmix_next(state);
  for (int i = 0; i < 4; i++) hi.w[i] = splitmix_next(state);
  memcpy(&r2, FR.r2, 32);
  fe_mul(&FR, &lo, &lo, &r2);      /* lo * 2^256 */
  fe_mul(&FR, &hi, &hi, &r2);      /* hi * 2^256 */
  fe_mul(&FR, &hi, &hi, &r2);      /* hi * 2^512 = Montgomery form of hi * 2^256 */
  fe_add(&FR, out, &lo, &hi);
}

void oracle_g1_add(const jac* a, const jac* b, jac* out) {
  xyzz x, y;
  xyzz_from_jac(&x, a);
  xyzz_from_jac(&y, b);
  xyzz_add(&x, &y);
  jac_store_normalised(out, &x);
}
void oracle_g1_mul(const fe* scalar_mont, const jac* p, jac* out) {
  fe s;
  fe_from_mont(&FR, &s, scalar_mont);
  xyzz base, acc;
  xyzz_from_jac(&base, p);
  xyzz_set_inf(&acc);
  for (int i = 3; i >= 0; i--)
    for (int b = 63; b >= 0; b--) {
      xyzz_dbl(&acc, &acc);
      if ((s.w[i] >> b) & 1) xyzz_add(&acc, &base);
    }
  jac_store_normalised(out, &acc);
}
int oracle_g1_eq(const jac* a, const jac* b) {
  xyzz x, y;
  jac na, nb;
  xyzz_from_jac(&x, a);
  xyzz_from_jac(&y, b);
  jac_store_normalised(&na, &x);
  jac_store_normalised(&nb, &y);
  return memcmp(&na, &nb, sizeof(jac)) == 0;
}
void oracle_g1_generator(jac* out) {
  fe one = {{1, 0, 0, 0}}, two = {{2, 0, 0, 0}};
  fe_to_mont(&FP, &out->x, &one);
  fe_to_mont(&FP, &out->y, &two);
  memcpy(&out->z, FP.one, 32);
}
