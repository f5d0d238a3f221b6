// Montgomery arithmetic for the two 254-bit BN254 prime fields on 8 x 32-bit limbs, written for
// the integer pipe of sm_100a (mad.lo.cc / madc.hi.cc carry chains that the assembler pairs into
// wide multiply-adds).
//
// Element layout is the reference's (include/field/mont_t.cuh:30-36, alt_bn128.cuh:53-73): eight
// little-endian 32-bit limbs holding value * 2^256 mod m, always fully reduced in memory.
//
// The multiplication is an operand-scanning Montgomery product that keeps the running value as
// two interleaved accumulators ("E" collects the products whose low word lands on an even limb,
// "O" the ones that land on an odd limb).  Each accumulator is extended by one pure carry chain
// per step, so no product ever has to be split across two chains.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#ifndef GRAPE_MUL_ATTR
#define GRAPE_MUL_ATTR __forceinline__
#endif

namespace grape {

// ---------------------------------------------------------------------------------------------
// Field parameters.  MOD: modulus, R2: 2^512 mod m, ONE: 2^256 mod m, M0: -m^-1 mod 2^32.
// ---------------------------------------------------------------------------------------------
struct FpParams {  // base field of BN254 (reference: ALT_BN128_P, include/field/alt_bn128.cuh:11-27)
  __host__ __device__ static constexpr uint32_t mod(int i) {
    constexpr uint32_t t[8] = {0xd87cfd47u, 0x3c208c16u, 0x6871ca8du, 0x97816a91u,
                                      0x8181585du, 0xb85045b6u, 0xe131a029u, 0x30644e72u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t r2(int i) {
    constexpr uint32_t t[8] = {0x538afa89u, 0xf32cfc5bu, 0xd44501fbu, 0xb5e71911u,
                                     0x0a417ff6u, 0x47ab1effu, 0xcab8351fu, 0x06d89f71u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t one(int i) {
    constexpr uint32_t t[8] = {0xc58f0d9du, 0xd35d438du, 0xf5c70b3du, 0x0a78eb28u,
                                      0x7879462cu, 0x666ea36fu, 0x9a07df2fu, 0x0e0a77c1u};
    return t[i];
  }
  static constexpr uint32_t M0 = 0xe4866389u;
};

struct FrParams {  // scalar field of BN254 (reference: ALT_BN128_r, include/field/alt_bn128.cuh:29-45)
  __host__ __device__ static constexpr uint32_t mod(int i) {
    constexpr uint32_t t[8] = {0xf0000001u, 0x43e1f593u, 0x79b97091u, 0x2833e848u,
                                      0x8181585du, 0xb85045b6u, 0xe131a029u, 0x30644e72u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t r2(int i) {
    constexpr uint32_t t[8] = {0xae216da7u, 0x1bb8e645u, 0xe35c59e3u, 0x53fe3ab1u,
                                     0x53bb8085u, 0x8c49833du, 0x7f4e44a5u, 0x0216d0b1u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t one(int i) {
    constexpr uint32_t t[8] = {0x4ffffffbu, 0xac96341cu, 0x9f60cd29u, 0x36fc7695u,
                                      0x7879462eu, 0x666ea36fu, 0x9a07df2fu, 0x0e0a77c1u};
    return t[i];
  }
  static constexpr uint32_t M0 = 0xefffffffu;
};

// ---------------------------------------------------------------------------------------------
// Carry-chain building blocks.  Every chain lives inside ONE asm statement so that the carry flag
// never has to survive across statements.
// ---------------------------------------------------------------------------------------------

// t[0..7] = {s0,s1,s2,s3} * b laid out as four adjacent 64-bit products (no carries needed).
__device__ __forceinline__ void mul4(uint32_t (&t)[8], uint32_t s0, uint32_t s1, uint32_t s2,
                                     uint32_t s3, uint32_t b) {
  asm("mul.lo.u32 %0, %8, %12;\n\t"
      "mul.hi.u32 %1, %8, %12;\n\t"
      "mul.lo.u32 %2, %9, %12;\n\t"
      "mul.hi.u32 %3, %9, %12;\n\t"
      "mul.lo.u32 %4, %10, %12;\n\t"
      "mul.hi.u32 %5, %10, %12;\n\t"
      "mul.lo.u32 %6, %11, %12;\n\t"
      "mul.hi.u32 %7, %11, %12;"
      : "=&r"(t[0]), "=&r"(t[1]), "=&r"(t[2]), "=&r"(t[3]), "=&r"(t[4]), "=&r"(t[5]), "=&r"(t[6]),
        "=&r"(t[7])
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(b));
}

// t[0..7] += {s0,s1,s2,s3} * b (one carry chain); the carry out of limb 7 is added to `top`.
__device__ __forceinline__ void mad4_top(uint32_t (&t)[8], uint32_t& top, uint32_t s0, uint32_t s1,
                                         uint32_t s2, uint32_t s3, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %9, %13, %0;\n\t"
      "madc.hi.cc.u32 %1, %9, %13, %1;\n\t"
      "madc.lo.cc.u32 %2, %10, %13, %2;\n\t"
      "madc.hi.cc.u32 %3, %10, %13, %3;\n\t"
      "madc.lo.cc.u32 %4, %11, %13, %4;\n\t"
      "madc.hi.cc.u32 %5, %11, %13, %5;\n\t"
      "madc.lo.cc.u32 %6, %12, %13, %6;\n\t"
      "madc.hi.cc.u32 %7, %12, %13, %7;\n\t"
      "addc.u32 %8, %8, 0;"
      : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]),
        "+r"(t[7]), "+r"(top)
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(b));
}

// Same without a carry out (used where the bound on the running value rules one out).
__device__ __forceinline__ void mad4(uint32_t (&t)[8], uint32_t s0, uint32_t s1, uint32_t s2,
                                     uint32_t s3, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %8, %12, %0;\n\t"
      "madc.hi.cc.u32 %1, %8, %12, %1;\n\t"
      "madc.lo.cc.u32 %2, %9, %12, %2;\n\t"
      "madc.hi.cc.u32 %3, %9, %12, %3;\n\t"
      "madc.lo.cc.u32 %4, %10, %12, %4;\n\t"
      "madc.hi.cc.u32 %5, %10, %12, %5;\n\t"
      "madc.lo.cc.u32 %6, %11, %12, %6;\n\t"
      "madc.hi.u32 %7, %11, %12, %7;"
      : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]),
        "+r"(t[7])
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(b));
}

// The step that divides the running value by 2^32 and adds the next odd-limb products in one go:
//   lo0 += e[1]                       (the only word of E that still sits below the new origin)
//   n[k] = e[k+2] + {s0..s3} * b      (carry in from the line above; e[8], e[9] read as zero)
__device__ __forceinline__ void shift_mad4(uint32_t (&n)[8], uint32_t& lo0, const uint32_t (&e)[8],
                                           uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3,
                                           uint32_t b) {
  asm("add.cc.u32 %8, %8, %9;\n\t"
      "madc.lo.cc.u32 %0, %16, %20, %10;\n\t"
      "madc.hi.cc.u32 %1, %16, %20, %11;\n\t"
      "madc.lo.cc.u32 %2, %17, %20, %12;\n\t"
      "madc.hi.cc.u32 %3, %17, %20, %13;\n\t"
      "madc.lo.cc.u32 %4, %18, %20, %14;\n\t"
      "madc.hi.cc.u32 %5, %18, %20, %15;\n\t"
      "madc.lo.cc.u32 %6, %19, %20, 0;\n\t"
      "madc.hi.u32 %7, %19, %20, 0;"
      : "=&r"(n[0]), "=&r"(n[1]), "=&r"(n[2]), "=&r"(n[3]), "=&r"(n[4]), "=&r"(n[5]), "=&r"(n[6]),
        "=&r"(n[7]), "+r"(lo0)
      : "r"(e[1]), "r"(e[2]), "r"(e[3]), "r"(e[4]), "r"(e[5]), "r"(e[6]), "r"(e[7]), "r"(s0),
        "r"(s1), "r"(s2), "r"(s3), "r"(b));
}

// r = a + b over 8 limbs, returns the carry out.
__device__ __forceinline__ uint32_t add8(uint32_t (&r)[8], const uint32_t (&a)[8],
                                         const uint32_t (&b)[8]) {
  uint32_t c;
  asm("add.cc.u32 %0, %9, %17;\n\t"
      "addc.cc.u32 %1, %10, %18;\n\t"
      "addc.cc.u32 %2, %11, %19;\n\t"
      "addc.cc.u32 %3, %12, %20;\n\t"
      "addc.cc.u32 %4, %13, %21;\n\t"
      "addc.cc.u32 %5, %14, %22;\n\t"
      "addc.cc.u32 %6, %15, %23;\n\t"
      "addc.cc.u32 %7, %16, %24;\n\t"
      "addc.u32 %8, 0, 0;"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]),
        "=&r"(r[7]), "=&r"(c)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]),
        "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]));
  return c;
}

// r = a - b over 8 limbs, returns 0xffffffff when the subtraction borrowed, else 0.
__device__ __forceinline__ uint32_t sub8(uint32_t (&r)[8], const uint32_t (&a)[8],
                                         const uint32_t (&b)[8]) {
  uint32_t m;
  asm("sub.cc.u32 %0, %9, %17;\n\t"
      "subc.cc.u32 %1, %10, %18;\n\t"
      "subc.cc.u32 %2, %11, %19;\n\t"
      "subc.cc.u32 %3, %12, %20;\n\t"
      "subc.cc.u32 %4, %13, %21;\n\t"
      "subc.cc.u32 %5, %14, %22;\n\t"
      "subc.cc.u32 %6, %15, %23;\n\t"
      "subc.cc.u32 %7, %16, %24;\n\t"
      "subc.u32 %8, 0, 0;"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]),
        "=&r"(r[7]), "=&r"(m)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]),
        "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]));
  return m;
}

// ---------------------------------------------------------------------------------------------
// Field element
// ---------------------------------------------------------------------------------------------
template <class PARAMS>
struct __align__(16) Fe {
  uint32_t v[8];
  using Params = PARAMS;

  __device__ __forceinline__ static void mod_limbs(uint32_t (&m)[8]) {
#pragma unroll
    for (int i = 0; i < 8; i++) m[i] = PARAMS::mod(i);
  }
  __device__ __forceinline__ static Fe zero() {
    Fe r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = 0;
    return r;
  }
  __device__ __forceinline__ static Fe one() {
    Fe r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = PARAMS::one(i);
    return r;
  }
  __device__ __forceinline__ static Fe r2() {
    Fe r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = PARAMS::r2(i);
    return r;
  }
  __device__ __forceinline__ bool is_zero() const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) o |= v[i];
    return o == 0;
  }
  __device__ __forceinline__ bool operator==(const Fe& b) const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) o |= v[i] ^ b.v[i];
    return o == 0;
  }
  __device__ __forceinline__ bool operator!=(const Fe& b) const { return !(*this == b); }

  // Loads / stores as two 16-byte vectors.
  __device__ __forceinline__ static Fe load(const void* p) {
    Fe r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
    uint4 a = q[0], b = q[1];
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
    return r;
  }
  __device__ __forceinline__ static Fe load_nc(const void* p) {
    Fe r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
    uint4 a = __ldg(q), b = __ldg(q + 1);
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
    return r;
  }
  __device__ __forceinline__ void store(void* p) const {
    uint4* q = reinterpret_cast<uint4*>(p);
    q[0] = make_uint4(v[0], v[1], v[2], v[3]);
    q[1] = make_uint4(v[4], v[5], v[6], v[7]);
  }
};

// r = a + b mod m
template <class P>
__device__ __forceinline__ Fe<P> fe_add(const Fe<P>& a, const Fe<P>& b) {
  uint32_t s[8], t[8], m[8];
  Fe<P>::mod_limbs(m);
  add8(s, a.v, b.v);  // both < m < 2^254: cannot carry out
  uint32_t borrow = sub8(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = borrow ? s[i] : t[i];
  return r;
}

// r = a - b mod m
template <class P>
__device__ __forceinline__ Fe<P> fe_sub(const Fe<P>& a, const Fe<P>& b) {
  uint32_t s[8], t[8], m[8];
  Fe<P>::mod_limbs(m);
  uint32_t borrow = sub8(s, a.v, b.v);
#pragma unroll
  for (int i = 0; i < 8; i++) m[i] &= borrow;
  add8(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = t[i];
  return r;
}

// r = -a mod m (0 stays 0)
template <class P>
__device__ __forceinline__ Fe<P> fe_neg(const Fe<P>& a) {
  uint32_t m[8], t[8];
  Fe<P>::mod_limbs(m);
  sub8(t, m, a.v);
  bool z = a.is_zero();
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = z ? 0u : t[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_cneg(const Fe<P>& a, bool flag) {
  Fe<P> n = fe_neg(a);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = flag ? n.v[i] : a.v[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_dbl(const Fe<P>& a) { return fe_add(a, a); }

// One reduction step shared by the multiplication and by leaving Montgomery form:
// adds mi * MOD so that limb 0 of E cancels.
template <class P>
__device__ __forceinline__ void redc_step(uint32_t (&E)[8], uint32_t (&O)[8]) {
  uint32_t mi = E[0] * P::M0;
  mad4(O, P::mod(1), P::mod(3), P::mod(5), P::mod(7), mi);
  mad4_top(E, O[7], P::mod(0), P::mod(2), P::mod(4), P::mod(6), mi);
}

// Final merge: value = (E >> 32) + O, then one conditional subtraction.
template <class P>
__device__ __forceinline__ Fe<P> mont_finish(const uint32_t (&E)[8], const uint32_t (&O)[8]) {
  uint32_t hi[8], s[8], t[8], m[8];
#pragma unroll
  for (int i = 0; i < 7; i++) hi[i] = E[i + 1];
  hi[7] = 0;
  add8(s, hi, O);
  Fe<P>::mod_limbs(m);
  uint32_t borrow = sub8(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = borrow ? s[i] : t[i];
  return r;
}

// r = a * b / 2^256 mod m
template <class P>
__device__ GRAPE_MUL_ATTR Fe<P> fe_mul(const Fe<P>& a, const Fe<P>& b) {
  uint32_t E[8], O[8];
  mul4(E, a.v[0], a.v[2], a.v[4], a.v[6], b.v[0]);
  mul4(O, a.v[1], a.v[3], a.v[5], a.v[7], b.v[0]);
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < 8; i++) {
    uint32_t N[8];
    // divide by 2^32: O becomes the even accumulator, E[2..] + odd products the new odd one
    shift_mad4(N, O[0], E, a.v[1], a.v[3], a.v[5], a.v[7], b.v[i]);
    mad4_top(O, N[7], a.v[0], a.v[2], a.v[4], a.v[6], b.v[i]);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      E[k] = O[k];
      O[k] = N[k];
    }
    redc_step<P>(E, O);
  }
  return mont_finish<P>(E, O);
}

template <class P>
__device__ __forceinline__ Fe<P> fe_sqr(const Fe<P>& a) { return fe_mul(a, a); }

// Leave Montgomery form: a / 2^256 mod m (eight reduction steps on the bare value).
template <class P>
__device__ __forceinline__ Fe<P> fe_from_mont(const Fe<P>& a) {
  uint32_t E[8], O[8];
#pragma unroll
  for (int i = 0; i < 8; i++) { E[i] = a.v[i]; O[i] = 0; }
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < 8; i++) {
    uint32_t N[8];
    shift_mad4(N, O[0], E, 0u, 0u, 0u, 0u, 0u);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      E[k] = O[k];
      O[k] = N[k];
    }
    redc_step<P>(E, O);
  }
  return mont_finish<P>(E, O);
}

// Enter Montgomery form: a * 2^256 mod m for any 256-bit a (the product with R^2 reduces it).
template <class P>
__device__ __forceinline__ Fe<P> fe_to_mont(const Fe<P>& a) { return fe_mul(a, Fe<P>::r2()); }

// a^(m-2) by square-and-multiply over the constant exponent (a = 0 maps to 0).
template <class P>
__device__ __noinline__ Fe<P> fe_inv(const Fe<P>& a) {
  uint32_t e[8];
#pragma unroll
  for (int i = 0; i < 8; i++) e[i] = P::mod(i);
  e[0] -= 2;  // MOD[0] >= 2 for both fields, no borrow
  Fe<P> acc = Fe<P>::one();
  for (int w = 7; w >= 0; w--) {
    uint32_t word = e[w];
    for (int bit = 31; bit >= 0; bit--) {
      acc = fe_sqr(acc);
      if ((word >> bit) & 1u) acc = fe_mul(acc, a);
    }
  }
  return acc;
}

// Signed 32-bit integer -> Montgomery residue; negatives map to m - |x|
// (reference: int_to_fr, src/fr-tensor.cu:30-39).
template <class P>
__device__ __forceinline__ Fe<P> fe_from_i32(int32_t x) {
  Fe<P> t = Fe<P>::zero();
  uint32_t ax = x < 0 ? (0u - (uint32_t)x) : (uint32_t)x;
  t.v[0] = ax;
  t = fe_to_mont(t);
  return fe_cneg(t, x < 0);
}

template <class P>
__device__ __forceinline__ Fe<P> fe_from_u32(uint32_t x) {
  Fe<P> t = Fe<P>::zero();
  t.v[0] = x;
  return fe_to_mont(t);
}

template <class P>
__device__ __forceinline__ Fe<P> fe_shfl_xor(const Fe<P>& a, int lane_mask) {
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = __shfl_xor_sync(0xffffffffu, a.v[i], lane_mask);
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_shfl_down(const Fe<P>& a, int delta) {
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = __shfl_down_sync(0xffffffffu, a.v[i], delta);
  return r;
}

using Fp = Fe<FpParams>;
using Fr = Fe<FrParams>;

}  // namespace grape
