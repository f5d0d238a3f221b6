// Short-Weierstrass G1 point arithmetic (a = 0: BN254 y^2 = x^3 + 3, BLS12-381 y^2 = x^3 + 4; the
// formulas never use b) for the commitment kernels, generic over the coordinate field F.
//
// Record layouts follow the reference so buffers are interchangeable with it (sizes for BN254, whose
// coordinates are 32 B; BLS12-381 coordinates are 48 B and every record grows by 3/2):
//   affine   64 B  X|Y, Montgomery form, (0,0) is the point at infinity  (include/curve/affine_t.cuh:17-75)
//   jacobian 96 B  X|Y|Z, Z = 0 is infinity                              (include/curve/jacobian_t.cuh:10-60)
//   xyzz    128 B  X|Y|ZZZ|ZZ with x = X/ZZ, y = Y/ZZZ, ZZ = 0 is infinity (include/curve/xyzz_t.cuh:16-40)
// Accumulation runs in XYZZ coordinates: adding an affine point costs 8 multiplications and 2
// squarings, and every special case (either side at infinity, equal points, opposite points)
// is handled so the result is correct for arbitrary inputs.
#pragma once
#include "field.cuh"

namespace grape {

template <class F>
struct __align__(16) AffineT {
  F x, y;
  __device__ __forceinline__ bool is_inf() const { return x.is_zero() && y.is_zero(); }
  __device__ __forceinline__ static AffineT<F> inf() { return AffineT<F>{F::zero(), F::zero()}; }
  __device__ __forceinline__ static AffineT<F> load_nc(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return AffineT<F>{F::load_nc(c), F::load_nc(c + F::BYTES)};
  }
  __device__ __forceinline__ static AffineT<F> load(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return AffineT<F>{F::load(c), F::load(c + F::BYTES)};
  }
  __device__ __forceinline__ void store(void* p) const {
    char* c = reinterpret_cast<char*>(p);
    x.store(c);
    y.store(c + F::BYTES);
  }
};

template <class F>
struct __align__(16) JacobianT {
  F x, y, z;
};

template <class F>
struct __align__(16) XyzzT {
  F x, y, zzz, zz;

  __device__ __forceinline__ static XyzzT<F> inf() {
    return XyzzT<F>{F::zero(), F::zero(), F::zero(), F::zero()};
  }
  __device__ __forceinline__ bool is_inf() const { return zz.is_zero(); }
  __device__ __forceinline__ static XyzzT<F> from_affine(const AffineT<F>& p) {
    if (p.is_inf()) return inf();
    return XyzzT<F>{p.x, p.y, F::one(), F::one()};
  }
  __device__ __forceinline__ static XyzzT<F> load(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return XyzzT<F>{F::load(c), F::load(c + F::BYTES), F::load(c + 2 * F::BYTES), F::load(c + 3 * F::BYTES)};
  }
  __device__ __forceinline__ void store(void* p) const {
    char* c = reinterpret_cast<char*>(p);
    x.store(c);
    y.store(c + F::BYTES);
    zzz.store(c + 2 * F::BYTES);
    zz.store(c + 3 * F::BYTES);
  }
};

// 2 * (affine point), affine point finite.
template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_dbl_affine(const AffineT<F>& p) {
  F U = fe_dbl(p.y);
  F V = fe_sqr(U);
  F W = fe_mul(U, V);
  F S = fe_mul(p.x, V);
  F X2 = fe_sqr(p.x);
  F M = fe_add(fe_dbl(X2), X2);
  XyzzT<F> r;
  r.x = fe_sub(fe_sqr(M), fe_dbl(S));
  r.y = fe_sub(fe_mul(M, fe_sub(S, r.x)), fe_mul(W, p.y));
  r.zz = V;
  r.zzz = W;
  if (p.y.is_zero()) return XyzzT<F>::inf();  // order-2 point (none on this curve, kept for safety)
  return r;
}

// 2 * P
template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_dbl(const XyzzT<F>& p) {
  if (p.is_inf()) return p;
  F U = fe_dbl(p.y);
  F V = fe_sqr(U);
  F W = fe_mul(U, V);
  F S = fe_mul(p.x, V);
  F X2 = fe_sqr(p.x);
  F M = fe_add(fe_dbl(X2), X2);
  XyzzT<F> r;
  r.x = fe_sub(fe_sqr(M), fe_dbl(S));
  r.y = fe_sub(fe_mul(M, fe_sub(S, r.x)), fe_mul(W, p.y));
  r.zz = fe_mul(V, p.zz);
  r.zzz = fe_mul(W, p.zzz);
  return r;
}

// 2 * P with the field operations as calls (see fe_mul_call): for serial doubling loops.
template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_dbl_compact(const XyzzT<F>& p) {
  if (p.is_inf()) return p;
  F U = fe_dbl(p.y);
  F V = fe_sqr_call(U);
  F W = fe_mul_call(U, V);
  F S = fe_mul_call(p.x, V);
  F X2 = fe_sqr_call(p.x);
  F M = fe_add(fe_dbl(X2), X2);
  XyzzT<F> r;
  r.x = fe_sub(fe_sqr_call(M), fe_dbl(S));
  r.y = fe_sub(fe_mul_call(M, fe_sub(S, r.x)), fe_mul_call(W, p.y));
  r.zz = fe_mul_call(V, p.zz);
  r.zzz = fe_mul_call(W, p.zzz);
  return r;
}

// acc += q (both XYZZ), the field operations as calls.
template <class F>
__device__ __forceinline__ void xyzz_add_compact(XyzzT<F>& acc, const XyzzT<F>& q) {
  if (q.is_inf()) return;
  if (acc.is_inf()) {
    acc = q;
    return;
  }
  F U1 = fe_mul_call(acc.x, q.zz);
  F U2 = fe_mul_call(q.x, acc.zz);
  F S1 = fe_mul_call(acc.y, q.zzz);
  F S2 = fe_mul_call(q.y, acc.zzz);
  F Pd = fe_sub(U2, U1);
  F Rd = fe_sub(S2, S1);
  if (Pd.is_zero()) {
    if (Rd.is_zero()) acc = xyzz_dbl_compact(acc);
    else acc = XyzzT<F>::inf();
    return;
  }
  F PP = fe_sqr_call(Pd);
  F PPP = fe_mul_call(Pd, PP);
  F Q = fe_mul_call(U1, PP);
  F X3 = fe_sub(fe_sub(fe_sqr_call(Rd), PPP), fe_dbl(Q));
  F Y3 = fe_sub(fe_mul_call(Rd, fe_sub(Q, X3)), fe_mul_call(S1, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_mul_call(fe_mul_call(acc.zz, q.zz), PP);
  acc.zzz = fe_mul_call(fe_mul_call(acc.zzz, q.zzz), PPP);
}

// acc += q (q affine).  The rare cases branch; the common path is straight-line.
template <class F>
__device__ __forceinline__ void xyzz_madd(XyzzT<F>& acc, const AffineT<F>& q) {
  if (q.is_inf()) return;
  if (acc.is_inf()) {
    acc = XyzzT<F>{q.x, q.y, F::one(), F::one()};
    return;
  }
  F U2 = fe_mul(q.x, acc.zz);
  F S2 = fe_mul(q.y, acc.zzz);
  F Pd = fe_sub(U2, acc.x);
  F Rd = fe_sub(S2, acc.y);
  if (Pd.is_zero()) {
    if (Rd.is_zero()) acc = xyzz_dbl_affine(q);
    else acc = XyzzT<F>::inf();
    return;
  }
  F PP = fe_sqr(Pd);
  F PPP = fe_mul(Pd, PP);
  F Q = fe_mul(acc.x, PP);
  F X3 = fe_sub(fe_sub(fe_sqr(Rd), PPP), fe_dbl(Q));
  F Y3 = fe_sub(fe_mul(Rd, fe_sub(Q, X3)), fe_mul(acc.y, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_mul(acc.zz, PP);
  acc.zzz = fe_mul(acc.zzz, PPP);
}

// acc += q (q affine, canonical) with the accumulator's coordinates kept as LAZY residues in [0, 2 p):
// the same formulas, every product without its closing subtraction.  The inner loop of the commitment
// kernel runs on this; xyzz_canon brings an accumulator back before anything else reads it.
template <class F>
__device__ __forceinline__ void xyzz_madd_lazy(XyzzT<F>& acc, const AffineT<F>& q) {
  if (q.is_inf()) return;
  if (fe_lis_zero(acc.zz)) {
    acc = XyzzT<F>{q.x, q.y, F::one(), F::one()};
    return;
  }
  F U2 = fe_lmul(q.x, acc.zz);
  F S2 = fe_lmul(q.y, acc.zzz);
  F Pd = fe_lsub(U2, acc.x);
  F Rd = fe_lsub(S2, acc.y);
  if (fe_lis_zero(Pd)) {
    if (fe_lis_zero(Rd)) acc = xyzz_dbl_affine(q);
    else acc = XyzzT<F>::inf();
    return;
  }
  F PP = fe_lsqr(Pd);
  F PPP = fe_lmul(Pd, PP);
  F Q = fe_lmul(acc.x, PP);
  F X3 = fe_lsub(fe_lsub(fe_lsqr(Rd), PPP), fe_ladd(Q, Q));
  F Y3 = fe_lsub(fe_lmul(Rd, fe_lsub(Q, X3)), fe_lmul(acc.y, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_lmul(acc.zz, PP);
  acc.zzz = fe_lmul(acc.zzz, PPP);
}

template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_canon(const XyzzT<F>& p) {
  return XyzzT<F>{fe_canon(p.x), fe_canon(p.y), fe_canon(p.zzz), fe_canon(p.zz)};
}

// acc += q (both XYZZ)
template <class F>
__device__ __forceinline__ void xyzz_add(XyzzT<F>& acc, const XyzzT<F>& q) {
  if (q.is_inf()) return;
  if (acc.is_inf()) {
    acc = q;
    return;
  }
  F U1 = fe_mul(acc.x, q.zz);
  F U2 = fe_mul(q.x, acc.zz);
  F S1 = fe_mul(acc.y, q.zzz);
  F S2 = fe_mul(q.y, acc.zzz);
  F Pd = fe_sub(U2, U1);
  F Rd = fe_sub(S2, S1);
  if (Pd.is_zero()) {
    if (Rd.is_zero()) acc = xyzz_dbl(acc);
    else acc = XyzzT<F>::inf();
    return;
  }
  F PP = fe_sqr(Pd);
  F PPP = fe_mul(Pd, PP);
  F Q = fe_mul(U1, PP);
  F X3 = fe_sub(fe_sub(fe_sqr(Rd), PPP), fe_dbl(Q));
  F Y3 = fe_sub(fe_mul(Rd, fe_sub(Q, X3)), fe_mul(S1, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_mul(fe_mul(acc.zz, q.zz), PP);
  acc.zzz = fe_mul(fe_mul(acc.zzz, q.zzz), PPP);
}

template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_shfl_down(const XyzzT<F>& p, int delta) {
  return XyzzT<F>{fe_shfl_down(p.x, delta), fe_shfl_down(p.y, delta), fe_shfl_down(p.zzz, delta),
              fe_shfl_down(p.zz, delta)};
}

// Jacobian (any Z) -> XYZZ:  ZZ = Z^2, ZZZ = Z^3.
template <class F>
__device__ __forceinline__ XyzzT<F> xyzz_from_jacobian(const JacobianT<F>& j) {
  if (j.z.is_zero()) return XyzzT<F>::inf();
  F zz = fe_sqr(j.z);
  return XyzzT<F>{j.x, j.y, fe_mul(zz, j.z), zz};
}

// XYZZ -> affine (one inversion).
template <class F>
__device__ __forceinline__ AffineT<F> xyzz_to_affine(const XyzzT<F>& p) {
  if (p.is_inf()) return AffineT<F>::inf();
  F t = fe_inv(fe_mul(p.zz, p.zzz));
  F izz = fe_mul(t, p.zzz);
  F izzz = fe_mul(t, p.zz);
  return AffineT<F>{fe_mul(p.x, izz), fe_mul(p.y, izzz)};
}

// Canonical Jacobian record: (x, y, 1), or (1, 1, 0) for infinity.
template <class F>
__device__ __forceinline__ void store_jacobian_normalised(void* out, const AffineT<F>& a, bool inf) {
  char* c = reinterpret_cast<char*>(out);
  if (inf) {
    F::one().store(c);
    F::one().store(c + F::BYTES);
    F::zero().store(c + 2 * F::BYTES);
  } else {
    a.x.store(c);
    a.y.store(c + F::BYTES);
    F::one().store(c + 2 * F::BYTES);
  }
}

// Curve descriptors for the kernels that are generic over the curve: coordinate field, scalar field,
// identifier stored in a generator table, scalar width, and how many 128-thread blocks of the
// accumulation kernel should share an SM (the 12-limb field needs about 3/2 of the registers).
struct Bn254 {
  using F = Fp;
  using S = Fr;
  static constexpr uint32_t ID = 0;
  static constexpr uint32_t SCALAR_BITS = 254;
  static constexpr int MSM_BLOCKS = 4;
};
struct Bls12381 {
  using F = BlsFp;
  using S = BlsFr;
  static constexpr uint32_t ID = 1;
  static constexpr uint32_t SCALAR_BITS = 255;
#ifndef GRAPE_BLS_MSM_BLOCKS
#define GRAPE_BLS_MSM_BLOCKS 3
#endif
  static constexpr int MSM_BLOCKS = GRAPE_BLS_MSM_BLOCKS;
};

using Affine = AffineT<Fp>;
using Jacobian = JacobianT<Fp>;
using Xyzz = XyzzT<Fp>;

}  // namespace grape
