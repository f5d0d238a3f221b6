// BN254 G1 (y^2 = x^3 + 3) point arithmetic for the commitment kernels.
//
// Record layouts follow the reference so buffers are interchangeable with it:
//   affine   64 B  X|Y, Montgomery form, (0,0) is the point at infinity  (include/curve/affine_t.cuh:17-75)
//   jacobian 96 B  X|Y|Z, Z = 0 is infinity                              (include/curve/jacobian_t.cuh:10-60)
//   xyzz    128 B  X|Y|ZZZ|ZZ with x = X/ZZ, y = Y/ZZZ, ZZ = 0 is infinity (include/curve/xyzz_t.cuh:16-40)
// Accumulation runs in XYZZ coordinates: adding an affine point costs 8 multiplications and 2
// squarings, and every special case (either side at infinity, equal points, opposite points)
// is handled so the result is correct for arbitrary inputs.
#pragma once
#include "field.cuh"

namespace grape {

struct __align__(16) Affine {
  Fp x, y;
  __device__ __forceinline__ bool is_inf() const { return x.is_zero() && y.is_zero(); }
  __device__ __forceinline__ static Affine inf() { return Affine{Fp::zero(), Fp::zero()}; }
  __device__ __forceinline__ static Affine load_nc(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return Affine{Fp::load_nc(c), Fp::load_nc(c + 32)};
  }
  __device__ __forceinline__ static Affine load(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return Affine{Fp::load(c), Fp::load(c + 32)};
  }
  __device__ __forceinline__ void store(void* p) const {
    char* c = reinterpret_cast<char*>(p);
    x.store(c);
    y.store(c + 32);
  }
};

struct __align__(16) Jacobian {
  Fp x, y, z;
};

struct __align__(16) Xyzz {
  Fp x, y, zzz, zz;

  __device__ __forceinline__ static Xyzz inf() {
    return Xyzz{Fp::zero(), Fp::zero(), Fp::zero(), Fp::zero()};
  }
  __device__ __forceinline__ bool is_inf() const { return zz.is_zero(); }
  __device__ __forceinline__ static Xyzz from_affine(const Affine& p) {
    if (p.is_inf()) return inf();
    return Xyzz{p.x, p.y, Fp::one(), Fp::one()};
  }
  __device__ __forceinline__ static Xyzz load(const void* p) {
    const char* c = reinterpret_cast<const char*>(p);
    return Xyzz{Fp::load(c), Fp::load(c + 32), Fp::load(c + 64), Fp::load(c + 96)};
  }
  __device__ __forceinline__ void store(void* p) const {
    char* c = reinterpret_cast<char*>(p);
    x.store(c);
    y.store(c + 32);
    zzz.store(c + 64);
    zz.store(c + 96);
  }
};

// 2 * (affine point), affine point finite.
__device__ __forceinline__ Xyzz xyzz_dbl_affine(const Affine& p) {
  Fp U = fe_dbl(p.y);
  Fp V = fe_sqr(U);
  Fp W = fe_mul(U, V);
  Fp S = fe_mul(p.x, V);
  Fp X2 = fe_sqr(p.x);
  Fp M = fe_add(fe_dbl(X2), X2);
  Xyzz r;
  r.x = fe_sub(fe_sqr(M), fe_dbl(S));
  r.y = fe_sub(fe_mul(M, fe_sub(S, r.x)), fe_mul(W, p.y));
  r.zz = V;
  r.zzz = W;
  if (p.y.is_zero()) return Xyzz::inf();  // order-2 point (none on this curve, kept for safety)
  return r;
}

// 2 * P
__device__ __forceinline__ Xyzz xyzz_dbl(const Xyzz& p) {
  if (p.is_inf()) return p;
  Fp U = fe_dbl(p.y);
  Fp V = fe_sqr(U);
  Fp W = fe_mul(U, V);
  Fp S = fe_mul(p.x, V);
  Fp X2 = fe_sqr(p.x);
  Fp M = fe_add(fe_dbl(X2), X2);
  Xyzz r;
  r.x = fe_sub(fe_sqr(M), fe_dbl(S));
  r.y = fe_sub(fe_mul(M, fe_sub(S, r.x)), fe_mul(W, p.y));
  r.zz = fe_mul(V, p.zz);
  r.zzz = fe_mul(W, p.zzz);
  return r;
}

// acc += q (q affine).  The rare cases branch; the common path is straight-line.
__device__ __forceinline__ void xyzz_madd(Xyzz& acc, const Affine& q) {
  if (q.is_inf()) return;
  if (acc.is_inf()) {
    acc = Xyzz{q.x, q.y, Fp::one(), Fp::one()};
    return;
  }
  Fp U2 = fe_mul(q.x, acc.zz);
  Fp S2 = fe_mul(q.y, acc.zzz);
  Fp Pd = fe_sub(U2, acc.x);
  Fp Rd = fe_sub(S2, acc.y);
  if (Pd.is_zero()) {
    if (Rd.is_zero()) acc = xyzz_dbl_affine(q);
    else acc = Xyzz::inf();
    return;
  }
  Fp PP = fe_sqr(Pd);
  Fp PPP = fe_mul(Pd, PP);
  Fp Q = fe_mul(acc.x, PP);
  Fp X3 = fe_sub(fe_sub(fe_sqr(Rd), PPP), fe_dbl(Q));
  Fp Y3 = fe_sub(fe_mul(Rd, fe_sub(Q, X3)), fe_mul(acc.y, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_mul(acc.zz, PP);
  acc.zzz = fe_mul(acc.zzz, PPP);
}

// acc += q (both XYZZ)
__device__ __forceinline__ void xyzz_add(Xyzz& acc, const Xyzz& q) {
  if (q.is_inf()) return;
  if (acc.is_inf()) {
    acc = q;
    return;
  }
  Fp U1 = fe_mul(acc.x, q.zz);
  Fp U2 = fe_mul(q.x, acc.zz);
  Fp S1 = fe_mul(acc.y, q.zzz);
  Fp S2 = fe_mul(q.y, acc.zzz);
  Fp Pd = fe_sub(U2, U1);
  Fp Rd = fe_sub(S2, S1);
  if (Pd.is_zero()) {
    if (Rd.is_zero()) acc = xyzz_dbl(acc);
    else acc = Xyzz::inf();
    return;
  }
  Fp PP = fe_sqr(Pd);
  Fp PPP = fe_mul(Pd, PP);
  Fp Q = fe_mul(U1, PP);
  Fp X3 = fe_sub(fe_sub(fe_sqr(Rd), PPP), fe_dbl(Q));
  Fp Y3 = fe_sub(fe_mul(Rd, fe_sub(Q, X3)), fe_mul(S1, PPP));
  acc.x = X3;
  acc.y = Y3;
  acc.zz = fe_mul(fe_mul(acc.zz, q.zz), PP);
  acc.zzz = fe_mul(fe_mul(acc.zzz, q.zzz), PPP);
}

__device__ __forceinline__ Xyzz xyzz_shfl_down(const Xyzz& p, int delta) {
  return Xyzz{fe_shfl_down(p.x, delta), fe_shfl_down(p.y, delta), fe_shfl_down(p.zzz, delta),
              fe_shfl_down(p.zz, delta)};
}

// Jacobian (any Z) -> XYZZ:  ZZ = Z^2, ZZZ = Z^3.
__device__ __forceinline__ Xyzz xyzz_from_jacobian(const Jacobian& j) {
  if (j.z.is_zero()) return Xyzz::inf();
  Fp zz = fe_sqr(j.z);
  return Xyzz{j.x, j.y, fe_mul(zz, j.z), zz};
}

// XYZZ -> affine (one inversion).
__device__ __forceinline__ Affine xyzz_to_affine(const Xyzz& p) {
  if (p.is_inf()) return Affine::inf();
  Fp t = fe_inv(fe_mul(p.zz, p.zzz));
  Fp izz = fe_mul(t, p.zzz);
  Fp izzz = fe_mul(t, p.zz);
  return Affine{fe_mul(p.x, izz), fe_mul(p.y, izzz)};
}

// Canonical Jacobian record: (x, y, 1), or (1, 1, 0) for infinity.
__device__ __forceinline__ void store_jacobian_normalised(void* out, const Affine& a, bool inf) {
  char* c = reinterpret_cast<char*>(out);
  if (inf) {
    Fp::one().store(c);
    Fp::one().store(c + 32);
    Fp::zero().store(c + 64);
  } else {
    a.x.store(c);
    a.y.store(c + 32);
    Fp::one().store(c + 64);
  }
}

}  // namespace grape
