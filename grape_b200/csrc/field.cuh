// Montgomery arithmetic for prime fields on 8 or 12 x 32-bit limbs (the two 254-bit BN254 fields; the
// 381-bit base field and 255-bit scalar field of BLS12-381), written for the integer pipe of sm_100a
// (mad.lo.cc / madc.hi.cc carry chains that the assembler pairs into wide multiply-adds).
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
  static constexpr int LIMBS = 8;
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
  static constexpr int LIMBS = 8;
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


// BLS12-381: 381-bit base field on twelve limbs (radix 2^384) and 255-bit scalar field on eight
// (radix 2^256); the reference lists these constants in include/field/bls12-381.cuh:7-46.
struct BlsFpParams {  // base field of BLS12-381
  static constexpr int LIMBS = 12;
  __host__ __device__ static constexpr uint32_t mod(int i) {
    constexpr uint32_t t[12] = {0xffffaaabu, 0xb9feffffu, 0xb153ffffu, 0x1eabfffeu,
                                      0xf6b0f624u, 0x6730d2a0u, 0xf38512bfu, 0x64774b84u,
                                      0x434bacd7u, 0x4b1ba7b6u, 0x397fe69au, 0x1a0111eau};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t r2(int i) {
    constexpr uint32_t t[12] = {0x1c341746u, 0xf4df1f34u, 0x09d104f1u, 0x0a76e6a6u,
                                      0x4c95b6d5u, 0x8de5476cu, 0x939d83c0u, 0x67eb88a9u,
                                      0xb519952du, 0x9a793e85u, 0x92cae3aau, 0x11988fe5u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t one(int i) {
    constexpr uint32_t t[12] = {0x0002fffdu, 0x76090000u, 0xc40c0002u, 0xebf4000bu,
                                      0x53c758bau, 0x5f489857u, 0x70525745u, 0x77ce5853u,
                                      0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
    return t[i];
  }
  static constexpr uint32_t M0 = 0xfffcfffdu;
};

struct BlsFrParams {  // scalar field of BLS12-381
  static constexpr int LIMBS = 8;
  __host__ __device__ static constexpr uint32_t mod(int i) {
    constexpr uint32_t t[8] = {0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u,
                                      0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t r2(int i) {
    constexpr uint32_t t[8] = {0xf3f29c6du, 0xc999e990u, 0x87925c23u, 0x2b6cedcbu,
                                      0x7254398fu, 0x05d31496u, 0x9f59ff11u, 0x0748d9d9u};
    return t[i];
  }
  __host__ __device__ static constexpr uint32_t one(int i) {
    constexpr uint32_t t[8] = {0xfffffffeu, 0x00000001u, 0x00034802u, 0x5884b7fau,
                                      0xecbc4ff5u, 0x998c4fefu, 0xacc5056fu, 0x1824b159u};
    return t[i];
  }
  static constexpr uint32_t M0 = 0xffffffffu;
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

// Shorter rows for the squaring: t[0..2K-1] += {s0..} * b as one carry chain, the carry out of the last
// limb is added to `top` (the limb that follows the row).
__device__ __forceinline__ void mad1_top(uint32_t& t0, uint32_t& t1, uint32_t& top, uint32_t s0, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %3, %4, %0;\n\t"
      "madc.hi.cc.u32 %1, %3, %4, %1;\n\t"
      "addc.u32 %2, %2, 0;"
      : "+r"(t0), "+r"(t1), "+r"(top)
      : "r"(s0), "r"(b));
}
__device__ __forceinline__ void mad2_top(uint32_t& t0, uint32_t& t1, uint32_t& t2, uint32_t& t3, uint32_t& top,
                                         uint32_t s0, uint32_t s1, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %5, %7, %0;\n\t"
      "madc.hi.cc.u32 %1, %5, %7, %1;\n\t"
      "madc.lo.cc.u32 %2, %6, %7, %2;\n\t"
      "madc.hi.cc.u32 %3, %6, %7, %3;\n\t"
      "addc.u32 %4, %4, 0;"
      : "+r"(t0), "+r"(t1), "+r"(t2), "+r"(t3), "+r"(top)
      : "r"(s0), "r"(s1), "r"(b));
}
__device__ __forceinline__ void mad3_top(uint32_t& t0, uint32_t& t1, uint32_t& t2, uint32_t& t3, uint32_t& t4,
                                         uint32_t& t5, uint32_t& top, uint32_t s0, uint32_t s1, uint32_t s2,
                                         uint32_t b) {
  asm("mad.lo.cc.u32 %0, %7, %10, %0;\n\t"
      "madc.hi.cc.u32 %1, %7, %10, %1;\n\t"
      "madc.lo.cc.u32 %2, %8, %10, %2;\n\t"
      "madc.hi.cc.u32 %3, %8, %10, %3;\n\t"
      "madc.lo.cc.u32 %4, %9, %10, %4;\n\t"
      "madc.hi.cc.u32 %5, %9, %10, %5;\n\t"
      "addc.u32 %6, %6, 0;"
      : "+r"(t0), "+r"(t1), "+r"(t2), "+r"(t3), "+r"(t4), "+r"(t5), "+r"(top)
      : "r"(s0), "r"(s1), "r"(s2), "r"(b));
}
// t[0..5] = {s0,s1,s2} * b (three adjacent 64-bit products, no carries).
__device__ __forceinline__ void mul3(uint32_t& t0, uint32_t& t1, uint32_t& t2, uint32_t& t3, uint32_t& t4,
                                     uint32_t& t5, uint32_t s0, uint32_t s1, uint32_t s2, uint32_t b) {
  asm("mul.lo.u32 %0, %6, %9;\n\t"
      "mul.hi.u32 %1, %6, %9;\n\t"
      "mul.lo.u32 %2, %7, %9;\n\t"
      "mul.hi.u32 %3, %7, %9;\n\t"
      "mul.lo.u32 %4, %8, %9;\n\t"
      "mul.hi.u32 %5, %8, %9;"
      : "=&r"(t0), "=&r"(t1), "=&r"(t2), "=&r"(t3), "=&r"(t4), "=&r"(t5)
      : "r"(s0), "r"(s1), "r"(s2), "r"(b));
}
// t[0..15] = 2 * d[0..15] + (a_0^2, a_1^2, ..., a_7^2 laid out as eight adjacent 64-bit squares): the
// doubled off-diagonal part of a square plus its diagonal, one carry chain.  d must be below 2^511.
__device__ __forceinline__ void sqr_diag8(uint32_t (&t)[16], const uint32_t (&d)[16], const uint32_t (&a)[8]) {
  uint32_t h[16];
  h[0] = d[0] << 1;
#pragma unroll
  for (int i = 1; i < 16; i++) h[i] = __funnelshift_l(d[i - 1], d[i], 1);
  asm("mad.lo.cc.u32 %0, %16, %16, %24;\n\t"
      "madc.hi.cc.u32 %1, %16, %16, %25;\n\t"
      "madc.lo.cc.u32 %2, %17, %17, %26;\n\t"
      "madc.hi.cc.u32 %3, %17, %17, %27;\n\t"
      "madc.lo.cc.u32 %4, %18, %18, %28;\n\t"
      "madc.hi.cc.u32 %5, %18, %18, %29;\n\t"
      "madc.lo.cc.u32 %6, %19, %19, %30;\n\t"
      "madc.hi.cc.u32 %7, %19, %19, %31;\n\t"
      "madc.lo.cc.u32 %8, %20, %20, %32;\n\t"
      "madc.hi.cc.u32 %9, %20, %20, %33;\n\t"
      "madc.lo.cc.u32 %10, %21, %21, %34;\n\t"
      "madc.hi.cc.u32 %11, %21, %21, %35;\n\t"
      "madc.lo.cc.u32 %12, %22, %22, %36;\n\t"
      "madc.hi.cc.u32 %13, %22, %22, %37;\n\t"
      "madc.lo.cc.u32 %14, %23, %23, %38;\n\t"
      "madc.hi.u32 %15, %23, %23, %39;"
      : "=&r"(t[0]), "=&r"(t[1]), "=&r"(t[2]), "=&r"(t[3]), "=&r"(t[4]), "=&r"(t[5]), "=&r"(t[6]), "=&r"(t[7]),
        "=&r"(t[8]), "=&r"(t[9]), "=&r"(t[10]), "=&r"(t[11]), "=&r"(t[12]), "=&r"(t[13]), "=&r"(t[14]), "=&r"(t[15])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]),
        "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]),
        "r"(h[8]), "r"(h[9]), "r"(h[10]), "r"(h[11]), "r"(h[12]), "r"(h[13]), "r"(h[14]), "r"(h[15]));
}
// r[0..14] = a[0..14] + b[0..14] (the two off-diagonal accumulators of a square; the sum is below 2^480).
__device__ __forceinline__ void add15(uint32_t (&r)[16], const uint32_t (&a)[16], const uint32_t (&b)[16]) {
  asm("add.cc.u32 %0, %15, %30;\n\t"
      "addc.cc.u32 %1, %16, %31;\n\t"
      "addc.cc.u32 %2, %17, %32;\n\t"
      "addc.cc.u32 %3, %18, %33;\n\t"
      "addc.cc.u32 %4, %19, %34;\n\t"
      "addc.cc.u32 %5, %20, %35;\n\t"
      "addc.cc.u32 %6, %21, %36;\n\t"
      "addc.cc.u32 %7, %22, %37;\n\t"
      "addc.cc.u32 %8, %23, %38;\n\t"
      "addc.cc.u32 %9, %24, %39;\n\t"
      "addc.cc.u32 %10, %25, %40;\n\t"
      "addc.cc.u32 %11, %26, %41;\n\t"
      "addc.cc.u32 %12, %27, %42;\n\t"
      "addc.cc.u32 %13, %28, %43;\n\t"
      "addc.u32 %14, %29, %44;"
      : "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7]), "=&r"(r[8]),
        "=&r"(r[9]), "=&r"(r[10]), "=&r"(r[11]), "=&r"(r[12]), "=&r"(r[13]), "=&r"(r[14]), "=&r"(r[15])
      : "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
        "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]),
        "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(b[8]), "r"(b[9]),
        "r"(b[10]), "r"(b[11]), "r"(b[12]), "r"(b[13]), "r"(b[14]), "r"(b[15]));
  r[0] = 0;
}
// The division by 2^32 between two reduction steps when no new products come in:
//   lo0 += e[1];  n[k] = e[k+2] + carry  (e[8], e[9] read as zero)
__device__ __forceinline__ void shift_only8(uint32_t (&n)[8], uint32_t& lo0, const uint32_t (&e)[8]) {
  asm("add.cc.u32 %8, %8, %9;\n\t"
      "addc.cc.u32 %0, %10, 0;\n\t"
      "addc.cc.u32 %1, %11, 0;\n\t"
      "addc.cc.u32 %2, %12, 0;\n\t"
      "addc.cc.u32 %3, %13, 0;\n\t"
      "addc.cc.u32 %4, %14, 0;\n\t"
      "addc.cc.u32 %5, %15, 0;\n\t"
      "addc.u32 %6, 0, 0;\n\t"
      "mov.u32 %7, 0;"
      : "=&r"(n[0]), "=&r"(n[1]), "=&r"(n[2]), "=&r"(n[3]), "=&r"(n[4]), "=&r"(n[5]), "=&r"(n[6]), "=&r"(n[7]),
        "+r"(lo0)
      : "r"(e[1]), "r"(e[2]), "r"(e[3]), "r"(e[4]), "r"(e[5]), "r"(e[6]), "r"(e[7]));
}

// Twelve-limb counterparts of the helpers above (six products per chain).
__device__ __forceinline__ void mul6(uint32_t (&t)[12], uint32_t s0, uint32_t s1, uint32_t s2,
                                     uint32_t s3, uint32_t s4, uint32_t s5, uint32_t b) {
  asm("mul.lo.u32 %0, %12, %18;\n\t"
      "mul.hi.u32 %1, %12, %18;\n\t"
      "mul.lo.u32 %2, %13, %18;\n\t"
      "mul.hi.u32 %3, %13, %18;\n\t"
      "mul.lo.u32 %4, %14, %18;\n\t"
      "mul.hi.u32 %5, %14, %18;\n\t"
      "mul.lo.u32 %6, %15, %18;\n\t"
      "mul.hi.u32 %7, %15, %18;\n\t"
      "mul.lo.u32 %8, %16, %18;\n\t"
      "mul.hi.u32 %9, %16, %18;\n\t"
      "mul.lo.u32 %10, %17, %18;\n\t"
      "mul.hi.u32 %11, %17, %18;"
      : "=&r"(t[0]), "=&r"(t[1]), "=&r"(t[2]), "=&r"(t[3]), "=&r"(t[4]), "=&r"(t[5]), "=&r"(t[6]), "=&r"(t[7]), "=&r"(t[8]), "=&r"(t[9]), "=&r"(t[10]), "=&r"(t[11])
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(s4), "r"(s5), "r"(b));
}

__device__ __forceinline__ void mad6_top(uint32_t (&t)[12], uint32_t& top, uint32_t s0, uint32_t s1, uint32_t s2,
    uint32_t s3, uint32_t s4, uint32_t s5, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %13, %19, %0;\n\t"
      "madc.hi.cc.u32 %1, %13, %19, %1;\n\t"
      "madc.lo.cc.u32 %2, %14, %19, %2;\n\t"
      "madc.hi.cc.u32 %3, %14, %19, %3;\n\t"
      "madc.lo.cc.u32 %4, %15, %19, %4;\n\t"
      "madc.hi.cc.u32 %5, %15, %19, %5;\n\t"
      "madc.lo.cc.u32 %6, %16, %19, %6;\n\t"
      "madc.hi.cc.u32 %7, %16, %19, %7;\n\t"
      "madc.lo.cc.u32 %8, %17, %19, %8;\n\t"
      "madc.hi.cc.u32 %9, %17, %19, %9;\n\t"
      "madc.lo.cc.u32 %10, %18, %19, %10;\n\t"
      "madc.hi.cc.u32 %11, %18, %19, %11;\n\t"
      "addc.u32 %12, %12, 0;"
      : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]), "+r"(t[8]), "+r"(t[9]), "+r"(t[10]), "+r"(t[11]), "+r"(top)
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(s4), "r"(s5), "r"(b));
}

__device__ __forceinline__ void mad6(uint32_t (&t)[12], uint32_t s0, uint32_t s1, uint32_t s2,
    uint32_t s3, uint32_t s4, uint32_t s5, uint32_t b) {
  asm("mad.lo.cc.u32 %0, %12, %18, %0;\n\t"
      "madc.hi.cc.u32 %1, %12, %18, %1;\n\t"
      "madc.lo.cc.u32 %2, %13, %18, %2;\n\t"
      "madc.hi.cc.u32 %3, %13, %18, %3;\n\t"
      "madc.lo.cc.u32 %4, %14, %18, %4;\n\t"
      "madc.hi.cc.u32 %5, %14, %18, %5;\n\t"
      "madc.lo.cc.u32 %6, %15, %18, %6;\n\t"
      "madc.hi.cc.u32 %7, %15, %18, %7;\n\t"
      "madc.lo.cc.u32 %8, %16, %18, %8;\n\t"
      "madc.hi.cc.u32 %9, %16, %18, %9;\n\t"
      "madc.lo.cc.u32 %10, %17, %18, %10;\n\t"
      "madc.hi.u32 %11, %17, %18, %11;"
      : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]), "+r"(t[8]), "+r"(t[9]), "+r"(t[10]), "+r"(t[11])
      : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(s4), "r"(s5), "r"(b));
}

__device__ __forceinline__ void shift_mad6(uint32_t (&n)[12], uint32_t& lo0, const uint32_t (&e)[12],
    uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3, uint32_t s4, uint32_t s5, uint32_t b) {
  asm("add.cc.u32 %12, %12, %13;\n\t"
      "madc.lo.cc.u32 %0, %24, %30, %14;\n\t"
      "madc.hi.cc.u32 %1, %24, %30, %15;\n\t"
      "madc.lo.cc.u32 %2, %25, %30, %16;\n\t"
      "madc.hi.cc.u32 %3, %25, %30, %17;\n\t"
      "madc.lo.cc.u32 %4, %26, %30, %18;\n\t"
      "madc.hi.cc.u32 %5, %26, %30, %19;\n\t"
      "madc.lo.cc.u32 %6, %27, %30, %20;\n\t"
      "madc.hi.cc.u32 %7, %27, %30, %21;\n\t"
      "madc.lo.cc.u32 %8, %28, %30, %22;\n\t"
      "madc.hi.cc.u32 %9, %28, %30, %23;\n\t"
      "madc.lo.cc.u32 %10, %29, %30, 0;\n\t"
      "madc.hi.u32 %11, %29, %30, 0;"
      : "=&r"(n[0]), "=&r"(n[1]), "=&r"(n[2]), "=&r"(n[3]), "=&r"(n[4]), "=&r"(n[5]), "=&r"(n[6]), "=&r"(n[7]), "=&r"(n[8]), "=&r"(n[9]), "=&r"(n[10]), "=&r"(n[11]), "+r"(lo0)
      : "r"(e[1]), "r"(e[2]), "r"(e[3]), "r"(e[4]), "r"(e[5]), "r"(e[6]), "r"(e[7]), "r"(e[8]), "r"(e[9]), "r"(e[10]), "r"(e[11]), "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(s4), "r"(s5), "r"(b));
}

__device__ __forceinline__ uint32_t add12(uint32_t (&r)[12], const uint32_t (&a)[12],
                                          const uint32_t (&b)[12]) {
  uint32_t c;
  asm("add.cc.u32 %0, %13, %25;\n\t"
      "addc.cc.u32 %1, %14, %26;\n\t"
      "addc.cc.u32 %2, %15, %27;\n\t"
      "addc.cc.u32 %3, %16, %28;\n\t"
      "addc.cc.u32 %4, %17, %29;\n\t"
      "addc.cc.u32 %5, %18, %30;\n\t"
      "addc.cc.u32 %6, %19, %31;\n\t"
      "addc.cc.u32 %7, %20, %32;\n\t"
      "addc.cc.u32 %8, %21, %33;\n\t"
      "addc.cc.u32 %9, %22, %34;\n\t"
      "addc.cc.u32 %10, %23, %35;\n\t"
      "addc.cc.u32 %11, %24, %36;\n\t"
      "addc.u32 %12, 0, 0;"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7]), "=&r"(r[8]), "=&r"(r[9]), "=&r"(r[10]), "=&r"(r[11]), "=&r"(c)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(b[8]), "r"(b[9]), "r"(b[10]), "r"(b[11]));
  return c;
}

__device__ __forceinline__ uint32_t sub12(uint32_t (&r)[12], const uint32_t (&a)[12],
                                          const uint32_t (&b)[12]) {
  uint32_t c;
  asm("sub.cc.u32 %0, %13, %25;\n\t"
      "subc.cc.u32 %1, %14, %26;\n\t"
      "subc.cc.u32 %2, %15, %27;\n\t"
      "subc.cc.u32 %3, %16, %28;\n\t"
      "subc.cc.u32 %4, %17, %29;\n\t"
      "subc.cc.u32 %5, %18, %30;\n\t"
      "subc.cc.u32 %6, %19, %31;\n\t"
      "subc.cc.u32 %7, %20, %32;\n\t"
      "subc.cc.u32 %8, %21, %33;\n\t"
      "subc.cc.u32 %9, %22, %34;\n\t"
      "subc.cc.u32 %10, %23, %35;\n\t"
      "subc.cc.u32 %11, %24, %36;\n\t"
      "subc.u32 %12, 0, 0;"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7]), "=&r"(r[8]), "=&r"(r[9]), "=&r"(r[10]), "=&r"(r[11]), "=&r"(c)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(b[8]), "r"(b[9]), "r"(b[10]), "r"(b[11]));
  return c;
}

// Size-generic front ends: PAR selects the even (0) or odd (1) limbs of `a` as the multiplicands.
template <int PAR>
__device__ __forceinline__ void mul_half(uint32_t (&t)[8], const uint32_t (&a)[8], uint32_t b) {
  mul4(t, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], b);
}
template <int PAR>
__device__ __forceinline__ void mul_half(uint32_t (&t)[12], const uint32_t (&a)[12], uint32_t b) {
  mul6(t, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], a[PAR + 8], a[PAR + 10], b);
}
template <int PAR>
__device__ __forceinline__ void mad_half(uint32_t (&t)[8], const uint32_t (&a)[8], uint32_t b) {
  mad4(t, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], b);
}
template <int PAR>
__device__ __forceinline__ void mad_half(uint32_t (&t)[12], const uint32_t (&a)[12], uint32_t b) {
  mad6(t, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], a[PAR + 8], a[PAR + 10], b);
}
template <int PAR>
__device__ __forceinline__ void mad_half_top(uint32_t (&t)[8], uint32_t& top, const uint32_t (&a)[8], uint32_t b) {
  mad4_top(t, top, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], b);
}
template <int PAR>
__device__ __forceinline__ void mad_half_top(uint32_t (&t)[12], uint32_t& top, const uint32_t (&a)[12], uint32_t b) {
  mad6_top(t, top, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], a[PAR + 8], a[PAR + 10], b);
}
template <int PAR>
__device__ __forceinline__ void shift_mad_half(uint32_t (&n)[8], uint32_t& lo0, const uint32_t (&e)[8],
                                               const uint32_t (&a)[8], uint32_t b) {
  shift_mad4(n, lo0, e, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], b);
}
template <int PAR>
__device__ __forceinline__ void shift_mad_half(uint32_t (&n)[12], uint32_t& lo0, const uint32_t (&e)[12],
                                               const uint32_t (&a)[12], uint32_t b) {
  shift_mad6(n, lo0, e, a[PAR], a[PAR + 2], a[PAR + 4], a[PAR + 6], a[PAR + 8], a[PAR + 10], b);
}
__device__ __forceinline__ uint32_t addn(uint32_t (&r)[8], const uint32_t (&a)[8], const uint32_t (&b)[8]) { return add8(r, a, b); }
__device__ __forceinline__ uint32_t addn(uint32_t (&r)[12], const uint32_t (&a)[12], const uint32_t (&b)[12]) { return add12(r, a, b); }
__device__ __forceinline__ uint32_t subn(uint32_t (&r)[8], const uint32_t (&a)[8], const uint32_t (&b)[8]) { return sub8(r, a, b); }
__device__ __forceinline__ uint32_t subn(uint32_t (&r)[12], const uint32_t (&a)[12], const uint32_t (&b)[12]) { return sub12(r, a, b); }

// ---------------------------------------------------------------------------------------------
// Field element
// ---------------------------------------------------------------------------------------------
template <class PARAMS>
struct __align__(16) Fe {
  static constexpr int N = PARAMS::LIMBS;   // 32-bit limbs (8 or 12)
  static constexpr int BYTES = 4 * N;
  uint32_t v[N];
  using Params = PARAMS;

  __device__ __forceinline__ static void mod_limbs(uint32_t (&m)[N]) {
#pragma unroll
    for (int i = 0; i < N; i++) m[i] = PARAMS::mod(i);
  }
  __device__ __forceinline__ static Fe zero() {
    Fe r;
#pragma unroll
    for (int i = 0; i < N; i++) r.v[i] = 0;
    return r;
  }
  __device__ __forceinline__ static Fe one() {
    Fe r;
#pragma unroll
    for (int i = 0; i < N; i++) r.v[i] = PARAMS::one(i);
    return r;
  }
  __device__ __forceinline__ static Fe r2() {
    Fe r;
#pragma unroll
    for (int i = 0; i < N; i++) r.v[i] = PARAMS::r2(i);
    return r;
  }
  __device__ __forceinline__ bool is_zero() const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < N; i++) o |= v[i];
    return o == 0;
  }
  __device__ __forceinline__ bool operator==(const Fe& b) const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < N; i++) o |= v[i] ^ b.v[i];
    return o == 0;
  }
  __device__ __forceinline__ bool operator!=(const Fe& b) const { return !(*this == b); }

  // Loads / stores as 16-byte vectors (two for 8 limbs, three for 12).
  __device__ __forceinline__ static Fe load(const void* p) {
    Fe r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int k = 0; k < N / 4; k++) {
      uint4 a = q[k];
      r.v[4 * k] = a.x; r.v[4 * k + 1] = a.y; r.v[4 * k + 2] = a.z; r.v[4 * k + 3] = a.w;
    }
    return r;
  }
  __device__ __forceinline__ static Fe load_nc(const void* p) {
    Fe r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int k = 0; k < N / 4; k++) {
      uint4 a = __ldg(q + k);
      r.v[4 * k] = a.x; r.v[4 * k + 1] = a.y; r.v[4 * k + 2] = a.z; r.v[4 * k + 3] = a.w;
    }
    return r;
  }
  __device__ __forceinline__ void store(void* p) const {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int k = 0; k < N / 4; k++) q[k] = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
  }
};

// r = a + b mod m
template <class P>
__device__ __forceinline__ Fe<P> fe_add(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  uint32_t s[N], t[N], m[N];
  Fe<P>::mod_limbs(m);
  addn(s, a.v, b.v);  // both operands < m < 2^(32 N - 1): cannot carry out
  uint32_t borrow = subn(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = borrow ? s[i] : t[i];
  return r;
}

// r = a - b mod m
template <class P>
__device__ __forceinline__ Fe<P> fe_sub(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  uint32_t s[N], t[N], m[N];
  Fe<P>::mod_limbs(m);
  uint32_t borrow = subn(s, a.v, b.v);
#pragma unroll
  for (int i = 0; i < N; i++) m[i] &= borrow;
  addn(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = t[i];
  return r;
}

// r = -a mod m (0 stays 0)
template <class P>
__device__ __forceinline__ Fe<P> fe_neg(const Fe<P>& a) {
  constexpr int N = P::LIMBS;
  uint32_t m[N], t[N];
  Fe<P>::mod_limbs(m);
  subn(t, m, a.v);
  bool z = a.is_zero();
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = z ? 0u : t[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_cneg(const Fe<P>& a, bool flag) {
  Fe<P> n = fe_neg(a);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < P::LIMBS; i++) r.v[i] = flag ? n.v[i] : a.v[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_dbl(const Fe<P>& a) { return fe_add(a, a); }

// One reduction step shared by the multiplication and by leaving Montgomery form:
// adds mi * MOD so that limb 0 of E cancels.
template <class P>
__device__ __forceinline__ void redc_step(uint32_t (&E)[P::LIMBS], uint32_t (&O)[P::LIMBS]) {
  constexpr int N = P::LIMBS;
  uint32_t m[N];
  Fe<P>::mod_limbs(m);
  uint32_t mi = E[0] * P::M0;
  mad_half<1>(O, m, mi);
  mad_half_top<0>(E, O[N - 1], m, mi);
}

// Final merge: value = (E >> 32) + O, then one conditional subtraction.
template <class P>
__device__ __forceinline__ Fe<P> mont_finish(const uint32_t (&E)[P::LIMBS], const uint32_t (&O)[P::LIMBS]) {
  constexpr int N = P::LIMBS;
  uint32_t hi[N], s[N], t[N], m[N];
#pragma unroll
  for (int i = 0; i < N - 1; i++) hi[i] = E[i + 1];
  hi[N - 1] = 0;
  addn(s, hi, O);
  Fe<P>::mod_limbs(m);
  uint32_t borrow = subn(t, s, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = borrow ? s[i] : t[i];
  return r;
}

// r = a * b / 2^(32 N) mod m.  Operands must be below 2^(32 N - 1) (true of every reduced element).
template <class P>
__device__ GRAPE_MUL_ATTR Fe<P> fe_mul(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  uint32_t E[N], O[N];
  mul_half<0>(E, a.v, b.v[0]);
  mul_half<1>(O, a.v, b.v[0]);
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < N; i++) {
    uint32_t Nx[N];
    // divide by 2^32: O becomes the even accumulator, E[2..] + odd products the new odd one
    shift_mad_half<1>(Nx, O[0], E, a.v, b.v[i]);
    mad_half_top<0>(O, Nx[N - 1], a.v, b.v[i]);
#pragma unroll
    for (int k = 0; k < N; k++) {
      E[k] = O[k];
      O[k] = Nx[k];
    }
    redc_step<P>(E, O);
  }
  return mont_finish<P>(E, O);
}

// r = a * a / 2^256 mod m for the eight-limb fields (reference: the dedicated squaring of
// include/field/mont_t.cuh:145-192).  The 28 off-diagonal limb products are formed once (rows of
// products whose low word lands on an even limb go to one accumulator, odd to another), doubled, and
// the 8 diagonal squares are added: 36 wide multiply-adds instead of 64.  The low half of the 512-bit
// square is then reduced by the eight steps the multiplication uses and the high half is added on:
//   (T + m p) / 2^256 = T_hi + (T_lo + m p) / 2^256 < 2 p.
template <class P, bool LAZY = false>
__device__ GRAPE_MUL_ATTR Fe<P> fe_sqr8(const Fe<P>& x) {
  static_assert(P::LIMBS == 8, "eight-limb fields only");
  const uint32_t (&a)[8] = x.v;
  uint32_t Ea[16], Oa[16];
#pragma unroll
  for (int i = 0; i < 16; i++) { Ea[i] = 0; Oa[i] = 0; }
  mul3(Ea[2], Ea[3], Ea[4], Ea[5], Ea[6], Ea[7], a[2], a[4], a[6], a[0]);
  mad3_top(Ea[4], Ea[5], Ea[6], Ea[7], Ea[8], Ea[9], Ea[10], a[3], a[5], a[7], a[1]);
  mad2_top(Ea[6], Ea[7], Ea[8], Ea[9], Ea[10], a[4], a[6], a[2]);
  mad2_top(Ea[8], Ea[9], Ea[10], Ea[11], Ea[12], a[5], a[7], a[3]);
  mad1_top(Ea[10], Ea[11], Ea[12], a[6], a[4]);
  mad1_top(Ea[12], Ea[13], Ea[14], a[7], a[5]);
  {
    uint32_t t[8];
    mul4(t, a[1], a[3], a[5], a[7], a[0]);
#pragma unroll
    for (int i = 0; i < 8; i++) Oa[1 + i] = t[i];
  }
  mad3_top(Oa[3], Oa[4], Oa[5], Oa[6], Oa[7], Oa[8], Oa[9], a[2], a[4], a[6], a[1]);
  mad3_top(Oa[5], Oa[6], Oa[7], Oa[8], Oa[9], Oa[10], Oa[11], a[3], a[5], a[7], a[2]);
  mad2_top(Oa[7], Oa[8], Oa[9], Oa[10], Oa[11], a[4], a[6], a[3]);
  mad2_top(Oa[9], Oa[10], Oa[11], Oa[12], Oa[13], a[5], a[7], a[4]);
  mad1_top(Oa[11], Oa[12], Oa[13], a[6], a[5]);
  mad1_top(Oa[13], Oa[14], Oa[15], a[7], a[6]);
  uint32_t D[16], T[16];
  add15(D, Ea, Oa);
  sqr_diag8(T, D, a);
  uint32_t E[8], O[8];
#pragma unroll
  for (int i = 0; i < 8; i++) { E[i] = T[i]; O[i] = 0; }
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < 8; i++) {
    uint32_t Nx[8];
    shift_only8(Nx, O[0], E);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      E[k] = O[k];
      O[k] = Nx[k];
    }
    redc_step<P>(E, O);
  }
  uint32_t hi[8], s[8], s2[8], t[8], m[8];
#pragma unroll
  for (int i = 0; i < 7; i++) hi[i] = E[i + 1];
  hi[7] = 0;
  add8(s, hi, O);
#pragma unroll
  for (int i = 0; i < 8; i++) hi[i] = T[8 + i];
  add8(s2, s, hi);  // below 2 p < 2^255: no carry out
  Fe<P> r;
  if (LAZY) {  // operands and result in [0, 2 m): (4 m^2 + 2^256 m) / 2^256 < 2 m
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = s2[i];
    return r;
  }
  Fe<P>::mod_limbs(m);
  uint32_t borrow = sub8(t, s2, m);
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = borrow ? s2[i] : t[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_sqr(const Fe<P>& a) {
#ifndef GRAPE_NO_DEDICATED_SQR
  if constexpr (P::LIMBS == 8) return fe_sqr8(a);
  else
#endif
    return fe_mul(a, a);
}

// ---------------------------------------------------------------------------------------------
// Lazy residues.  Where 4 m < 2^(32 N) (both curves' base fields: BN254 p < 2^254, BLS12-381 p < 2^381
// on twelve limbs) a value may be kept anywhere in [0, 2 m): the Montgomery product of two such values is
// below (4 m^2) / 2^(32 N) + m < 2 m WITHOUT the closing conditional subtraction, and sums / differences
// are brought back into [0, 2 m) by one conditional correction with 2 m.  The commitment inner loop runs
// on these (fe_lmul, fe_lsqr, fe_ladd, fe_lsub): each product sheds a subtract chain and a select chain.
// A value is zero mod m iff it is 0 or m (fe_lis_zero); fe_canon returns the canonical residue.
// ---------------------------------------------------------------------------------------------
template <class P>
__device__ __forceinline__ void mod2_limbs(uint32_t (&m2)[P::LIMBS]) {
  constexpr int N = P::LIMBS;
#pragma unroll
  for (int i = 0; i < N; i++) m2[i] = (P::mod(i) << 1) | (i ? (P::mod(i - 1) >> 31) : 0u);
}

template <class P>
__device__ __forceinline__ Fe<P> mont_finish_lazy(const uint32_t (&E)[P::LIMBS], const uint32_t (&O)[P::LIMBS]) {
  constexpr int N = P::LIMBS;
  uint32_t hi[N];
#pragma unroll
  for (int i = 0; i < N - 1; i++) hi[i] = E[i + 1];
  hi[N - 1] = 0;
  Fe<P> r;
  addn(r.v, hi, O);
  return r;
}

// a * b / 2^(32 N), operands in [0, 2 m), result in [0, 2 m)
template <class P>
__device__ GRAPE_MUL_ATTR Fe<P> fe_lmul(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  static_assert((P::mod(N - 1) >> 30) == 0, "lazy residues need 4 m < 2^(32 N)");
  uint32_t E[N], O[N];
  mul_half<0>(E, a.v, b.v[0]);
  mul_half<1>(O, a.v, b.v[0]);
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < N; i++) {
    uint32_t Nx[N];
    shift_mad_half<1>(Nx, O[0], E, a.v, b.v[i]);
    mad_half_top<0>(O, Nx[N - 1], a.v, b.v[i]);
#pragma unroll
    for (int k = 0; k < N; k++) {
      E[k] = O[k];
      O[k] = Nx[k];
    }
    redc_step<P>(E, O);
  }
  return mont_finish_lazy<P>(E, O);
}

template <class P>
__device__ __forceinline__ Fe<P> fe_lsqr(const Fe<P>& a) {
#ifndef GRAPE_NO_DEDICATED_SQR
  if constexpr (P::LIMBS == 8) return fe_sqr8<P, true>(a);
  else
#endif
    return fe_lmul(a, a);
}

template <class P>
__device__ __forceinline__ Fe<P> fe_ladd(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  uint32_t s[N], t[N], m2[N];
  mod2_limbs<P>(m2);
  addn(s, a.v, b.v);  // below 4 m: no carry out
  const uint32_t borrow = subn(t, s, m2);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = borrow ? s[i] : t[i];
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_lsub(const Fe<P>& a, const Fe<P>& b) {
  constexpr int N = P::LIMBS;
  uint32_t s[N], m2[N];
  mod2_limbs<P>(m2);
  const uint32_t borrow = subn(s, a.v, b.v);
#pragma unroll
  for (int i = 0; i < N; i++) m2[i] &= borrow;
  Fe<P> r;
  addn(r.v, s, m2);
  return r;
}

template <class P>
__device__ __forceinline__ bool fe_lis_zero(const Fe<P>& a) {
  uint32_t z = 0, e = 0;
#pragma unroll
  for (int i = 0; i < P::LIMBS; i++) {
    z |= a.v[i];
    e |= a.v[i] ^ P::mod(i);
  }
  return z == 0 || e == 0;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_canon(const Fe<P>& a) {
  constexpr int N = P::LIMBS;
  uint32_t t[N], m[N];
  Fe<P>::mod_limbs(m);
  const uint32_t borrow = subn(t, a.v, m);
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < N; i++) r.v[i] = borrow ? a.v[i] : t[i];
  return r;
}

// Leave Montgomery form: a / 2^(32 N) mod m (N reduction steps on the bare value).
template <class P>
__device__ __forceinline__ Fe<P> fe_from_mont(const Fe<P>& a) {
  constexpr int N = P::LIMBS;
  uint32_t E[N], O[N], Z[N];
#pragma unroll
  for (int i = 0; i < N; i++) { E[i] = a.v[i]; O[i] = 0; Z[i] = 0; }
  redc_step<P>(E, O);
#pragma unroll
  for (int i = 1; i < N; i++) {
    uint32_t Nx[N];
    shift_mad_half<1>(Nx, O[0], E, Z, 0u);
#pragma unroll
    for (int k = 0; k < N; k++) {
      E[k] = O[k];
      O[k] = Nx[k];
    }
    redc_step<P>(E, O);
  }
  return mont_finish<P>(E, O);
}

// Enter Montgomery form: a * 2^(32 N) mod m (the product with R^2 reduces it).
template <class P>
__device__ __forceinline__ Fe<P> fe_to_mont(const Fe<P>& a) { return fe_mul(a, Fe<P>::r2()); }

// a^(m-2) by square-and-multiply over the constant exponent (a = 0 maps to 0): about 1.5 * bits
// dependent multiplications.  Kept as the cross-check of fe_inv below.
template <class P>
__device__ __noinline__ Fe<P> fe_inv_fermat(const Fe<P>& a) {
  constexpr int N = P::LIMBS;
  uint32_t e[N];
#pragma unroll
  for (int i = 0; i < N; i++) e[i] = P::mod(i);
  // exponent m - 2, with the borrow carried (the low limb of the BLS12-381 scalar modulus is 1)
  uint32_t borrow = e[0] < 2u ? 1u : 0u;
  e[0] -= 2u;
#pragma unroll
  for (int i = 1; i < N; i++) {
    const uint32_t b = (e[i] < borrow) ? 1u : 0u;
    e[i] -= borrow;
    borrow = b;
  }
  Fe<P> acc = Fe<P>::one();
  for (int w = N - 1; w >= 0; w--) {
    uint32_t word = e[w];
    for (int bit = 31; bit >= 0; bit--) {
      acc = fe_sqr(acc);
      if ((word >> bit) & 1u) acc = fe_mul(acc, a);
    }
  }
  return acc;
}

// v >>= z over N limbs, 0 <= z <= 31
template <int N>
__device__ __forceinline__ void shr_var(uint32_t (&v)[N], uint32_t z) {
#pragma unroll
  for (int i = 0; i < N - 1; i++) v[i] = __funnelshift_r(v[i], v[i + 1], z);
  v[N - 1] >>= z;
}
// v <<= z over N limbs, 0 <= z <= 31 (the bits shifted out must be clear)
template <int N>
__device__ __forceinline__ void shl_var(uint32_t (&v)[N], uint32_t z) {
#pragma unroll
  for (int i = N - 1; i > 0; i--) v[i] = __funnelshift_l(v[i - 1], v[i], z);
  v[0] <<= z;
}
// trailing zeros of the low limb, at most 31 (an all-zero low limb counts as 31: the caller shifts again)
__device__ __forceinline__ uint32_t ctz_cap31(uint32_t lo) {
  return lo ? min((uint32_t)(__ffs((int)lo) - 1), 31u) : 31u;
}

// Montgomery inverse: for a = x * 2^(32 N) mod m returns x^-1 * 2^(32 N) mod m; 0 maps to 0.
// Binary extended Euclid in Kaliski's "almost inverse" form on (u, v, r, s) = (m, a, 0, 1): while both
// u and v are odd the smaller is subtracted from the larger, the companion pair gets r + s, and ALL
// the factors of two of the difference are shifted out at once (the companion of the other side is
// shifted up by as many bits), k counting the shifts.  The loop leaves r = -a^-1 * 2^k mod m with
// k in [bits, 2 bits], and two Montgomery products by powers of two take the 2^k out.  About 0.7
// iterations per bit, each a few add / shift chains on the plain integers with both outcomes of the
// comparison computed side by side and selected (no divergence inside a warp except at the exit):
// roughly a tenth of the dependent-instruction latency of the Fermat ladder.  The reference inverts
// with a Euclid as well (include/field/mont_t.cuh:1058-1120).
template <class P>
__device__ __noinline__ Fe<P> fe_inv_kaliski(const Fe<P>& a) {
  constexpr int N = P::LIMBS;
  if (a.is_zero()) return a;
  uint32_t u[N], v[N], r[N], s[N];
#pragma unroll
  for (int i = 0; i < N; i++) { u[i] = P::mod(i); v[i] = a.v[i]; r[i] = 0; s[i] = 0; }
  s[0] = 1;
  uint32_t k = 0;
  for (;;) {
    if ((u[0] & 1u) == 0) {  // only after a shift that was cut at 31 bits
      const uint32_t z = ctz_cap31(u[0]);
      shr_var<N>(u, z);
      shl_var<N>(s, z);
      k += z;
      continue;
    }
    if ((v[0] & 1u) == 0) {  // an even input, or after a shift that was cut at 31 bits (v is never 0 here)
      const uint32_t z = ctz_cap31(v[0]);
      shr_var<N>(v, z);
      shl_var<N>(r, z);
      k += z;
      continue;
    }
    uint32_t d1[N], d2[N], t[N];
    const uint32_t lt = subn(d1, u, v);  // all ones when u < v
    subn(d2, v, u);
    addn(t, r, s);
    uint32_t ad[N], nz = 0;
#pragma unroll
    for (int i = 0; i < N; i++) {
      ad[i] = lt ? d2[i] : d1[i];  // |u - v|, even
      nz |= ad[i];
    }
    if (nz == 0) {  // u == v == gcd = 1: the closing step v = 0, s += r, r *= 2
#pragma unroll
      for (int i = 0; i < N; i++) s[i] = t[i];
      shl_var<N>(r, 1);
      k += 1;
      break;
    }
    const uint32_t z = ctz_cap31(ad[0]);
    shr_var<N>(ad, z);
    uint32_t big[N];
#pragma unroll
    for (int i = 0; i < N; i++) big[i] = lt ? r[i] : s[i];
    shl_var<N>(big, z);
#pragma unroll
    for (int i = 0; i < N; i++) {
      u[i] = lt ? u[i] : ad[i];
      v[i] = lt ? ad[i] : v[i];
      r[i] = lt ? big[i] : t[i];
      s[i] = lt ? t[i] : big[i];
    }
    k += z;
  }
  // r < 2 m holds -a^-1 * 2^k: bring it below m and negate
  uint32_t m[N], t[N];
  Fe<P>::mod_limbs(m);
  uint32_t borrow = subn(t, r, m);
  Fe<P> x;
#pragma unroll
  for (int i = 0; i < N; i++) x.v[i] = borrow ? r[i] : t[i];
  x = fe_neg(x);
  // x = a^-1 * 2^k.  The result is a^-1 * 2^(64 N):  x * 2^(32 N) by a product with R^2, then
  // * 2^(32 N - k) by a product with the plain power of two 2^(64 N - k) (kept below 2^(32 N - 2):
  // the few excess doublings of a very short run are done modularly).
  x = fe_mul(x, Fe<P>::r2());
  uint32_t j = 64u * N - k;
  while (j > 32u * N - 2u) {
    x = fe_dbl(x);
    j--;
  }
  Fe<P> pw = Fe<P>::zero();
#pragma unroll
  for (int i = 0; i < N; i++) pw.v[i] = ((j >> 5) == (uint32_t)i) ? (1u << (j & 31u)) : 0u;
  return fe_mul(x, pw);
}

// ---------------------------------------------------------------------------------------------
// Inversion by batched division steps (D. J. Bernstein and B.-Y. Yang, "Fast constant-time gcd
// computation and modular inversion", 2019; the variable-time form).  A division step maps
//     (delta, f, g) -> (1 - delta, g, (g - f) / 2)          if delta > 0 and g is odd,
//                      (1 + delta, f, (g + (g mod 2) f) / 2)  otherwise,
// keeps f odd and drives g to 0, at which point f = +-gcd.  Thirty steps depend only on the low 30 bits
// of f and g, so they run on two 32-bit registers and produce a 2 x 2 integer matrix (entries up to
// 2^30) that is then applied once to the full-width f, g (exactly divisible by 2^30) and, modulo m with
// the division by 2^30 done by adding the right multiple of m, to the pair (d, e) that carries
// d a = f, e a = g (mod m).  About 19 batches for a 254-bit modulus instead of about 180 full-width
// compare / subtract / shift iterations of the Euclid above: a third of its instructions and far
// shorter dependency chains.  Values are held in limbs of 30 bits (signed 32-bit words, the top one
// carrying the sign) so that every product is one 32 x 32 -> 64-bit signed multiply-add.
// ---------------------------------------------------------------------------------------------
template <class P>
struct Divsteps {
  static constexpr int N = P::LIMBS;
  static constexpr int L = (32 * N + 2 + 29) / 30;                         // 9 limbs for 256 bits, 13 for 384
  static constexpr int MAX_BATCHES = ((49 * 32 * N + 57) / 17 + 29) / 30 + 1;  // proven bound on the steps, + 1
  static constexpr int32_t M30 = (1 << 30) - 1;
  // limb j of the modulus in 30-bit limbs
  __host__ __device__ static constexpr int32_t mod30(int j) {
    const int bit = 30 * j, w = bit >> 5, sh = bit & 31;
    const uint64_t lo = w < N ? P::mod(w) : 0u, hi = w + 1 < N ? P::mod(w + 1) : 0u;
    return (int32_t)((((hi << 32) | lo) >> sh) & (uint64_t)M30);
  }
  // m^-1 mod 2^30 (Newton: five doublings of precision from m0 * m0 = 1 mod 8)
  __host__ __device__ static constexpr uint32_t minv30() {
    const uint32_t m0 = P::mod(0);
    uint32_t x = m0;
    for (int k = 0; k < 5; k++) x *= 2u - m0 * x;
    return x & (uint32_t)M30;
  }
};

template <class P>
__device__ __noinline__ Fe<P> fe_inv(const Fe<P>& a) {
  using D = Divsteps<P>;
  constexpr int N = P::LIMBS, L = D::L;
  constexpr int32_t M30 = D::M30;
  if (a.is_zero()) return a;
  int32_t f[L], g[L], d[L], e[L];
#pragma unroll
  for (int j = 0; j < L; j++) {
    const int bit = 30 * j, w = bit >> 5, sh = bit & 31;
    const uint32_t lo = w < N ? a.v[w] : 0u, hi = w + 1 < N ? a.v[w + 1] : 0u;
    g[j] = (int32_t)(__funnelshift_r(lo, hi, sh) & (uint32_t)M30);
    f[j] = D::mod30(j);
    d[j] = 0;
    e[j] = 0;
  }
  e[0] = 1;
  int32_t delta = 1;
#pragma unroll 1
  for (int batch = 0; batch < D::MAX_BATCHES; batch++) {
    // thirty division steps on the low words; (u, v; q, r) maps (f, g) to 2^30 (f', g')
    uint32_t f0 = (uint32_t)f[0] | ((uint32_t)f[1] << 30), g0 = (uint32_t)g[0] | ((uint32_t)g[1] << 30);
    uint32_t u = 1, v = 0, q = 0, r = 1;
    int left = 30;
    for (;;) {
      const int z = __ffs((int)(g0 | (1u << left))) - 1;  // zero steps, at most what is left of the batch
      g0 >>= z;
      u <<= z;
      v <<= z;
      delta += z;
      left -= z;
      if (left == 0) break;
      if (delta > 0) {  // (f, g) <- (g, -f), then g <- g + f below: the (g - f) / 2 step
        delta = -delta;
        const uint32_t tf = f0, tu = u, tv = v;
        f0 = g0;
        g0 = 0u - tf;
        u = q;
        v = r;
        q = 0u - tu;
        r = 0u - tv;
      }
      g0 += f0;
      q += u;
      r += v;
    }
    const int64_t su = (int32_t)u, sv = (int32_t)v, sq = (int32_t)q, sr = (int32_t)r;
    // (f, g) <- (u f + v g, q f + r g) / 2^30, exact
    {
      int64_t cf = su * f[0] + sv * g[0], cg = sq * f[0] + sr * g[0];
      cf >>= 30;
      cg >>= 30;
#pragma unroll
      for (int j = 1; j < L; j++) {
        cf += su * f[j] + sv * g[j];
        cg += sq * f[j] + sr * g[j];
        f[j - 1] = (int32_t)cf & M30;
        g[j - 1] = (int32_t)cg & M30;
        cf >>= 30;
        cg >>= 30;
      }
      f[L - 1] = (int32_t)cf;
      g[L - 1] = (int32_t)cg;
    }
    // (d, e) <- (u d + v e + md m, q d + r e + me m) / 2^30 with d, e kept in (-2 m, m): md, me start
    // as the coefficients of the negative ones among d, e and are then lowered to the multiple of m that
    // clears the low 30 bits
    {
      const int32_t sd = d[L - 1] >> 31, se = e[L - 1] >> 31;
      int32_t md = ((int32_t)u & sd) + ((int32_t)v & se), me = ((int32_t)q & sd) + ((int32_t)r & se);
      int64_t cd = su * d[0] + sv * e[0], ce = sq * d[0] + sr * e[0];
      md -= (int32_t)((D::minv30() * (uint32_t)cd + (uint32_t)md) & (uint32_t)M30);
      me -= (int32_t)((D::minv30() * (uint32_t)ce + (uint32_t)me) & (uint32_t)M30);
      cd += (int64_t)D::mod30(0) * md;
      ce += (int64_t)D::mod30(0) * me;
      cd >>= 30;
      ce >>= 30;
#pragma unroll
      for (int j = 1; j < L; j++) {
        cd += su * d[j] + sv * e[j] + (int64_t)D::mod30(j) * md;
        ce += sq * d[j] + sr * e[j] + (int64_t)D::mod30(j) * me;
        d[j - 1] = (int32_t)cd & M30;
        e[j - 1] = (int32_t)ce & M30;
        cd >>= 30;
        ce >>= 30;
      }
      d[L - 1] = (int32_t)cd;
      e[L - 1] = (int32_t)ce;
    }
    int32_t nz = 0;
#pragma unroll
    for (int j = 0; j < L; j++) nz |= g[j];
    if (nz == 0) break;
  }
  // f = +-1 and d a = f: the inverse is d or -d, taken from (-2 m, m) into [0, m)
  auto carry = [&](int32_t (&x)[L]) {
    int32_t c = 0;
#pragma unroll
    for (int j = 0; j < L - 1; j++) {
      x[j] += c;
      c = x[j] >> 30;
      x[j] &= M30;
    }
    x[L - 1] += c;
  };
  {
    const int32_t sf = f[L - 1] >> 31;  // all ones when f = -1
#pragma unroll
    for (int j = 0; j < L; j++) d[j] = (d[j] ^ sf) - sf;
    carry(d);
  }
#pragma unroll 1
  for (int k = 0; k < 2; k++) {  // d in (-2 m, 2 m): at most two additions of m
    const int32_t neg = d[L - 1] >> 31;
#pragma unroll
    for (int j = 0; j < L; j++) d[j] += D::mod30(j) & neg;
    carry(d);
  }
  {
    int32_t t[L];
#pragma unroll
    for (int j = 0; j < L; j++) t[j] = d[j] - D::mod30(j);
    carry(t);
    const int32_t keep = t[L - 1] >> 31;  // all ones when d < m already
#pragma unroll
    for (int j = 0; j < L; j++) d[j] = (d[j] & keep) | (t[j] & ~keep);
  }
  Fe<P> x;
#pragma unroll
  for (int i = 0; i < N; i++) {
    const int bit = 32 * i, j = bit / 30, sh = bit % 30;
    uint64_t w = (uint64_t)(uint32_t)d[j] >> sh;
    if (j + 1 < L) w |= (uint64_t)(uint32_t)d[j + 1] << (30 - sh);
    if (j + 2 < L) w |= (uint64_t)(uint32_t)d[j + 2] << (60 - sh);
    x.v[i] = (uint32_t)w;
  }
  // x = a^-1 on the stored (Montgomery) value; the result is a^-1 * 2^(64 N)
  return fe_mul(fe_mul(x, Fe<P>::r2()), Fe<P>::r2());
}

// The multiplication and the squaring as real function calls, for code that runs as ONE serial
// instruction stream (a thread doubling a point a few hundred times): with every product inlined such a
// loop body is tens of kilobytes and the warp waits on instruction fetch as much as on arithmetic.
template <class P>
__device__ __noinline__ Fe<P> fe_mul_call(Fe<P> a, Fe<P> b) { return fe_mul(a, b); }  // by value: in registers
template <class P>
__device__ __noinline__ Fe<P> fe_sqr_call(Fe<P> a) { return fe_sqr(a); }

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
  for (int i = 0; i < P::LIMBS; i++) r.v[i] = __shfl_xor_sync(0xffffffffu, a.v[i], lane_mask);
  return r;
}

template <class P>
__device__ __forceinline__ Fe<P> fe_shfl_down(const Fe<P>& a, int delta) {
  Fe<P> r;
#pragma unroll
  for (int i = 0; i < P::LIMBS; i++) r.v[i] = __shfl_down_sync(0xffffffffu, a.v[i], delta);
  return r;
}

using Fp = Fe<FpParams>;
using Fr = Fe<FrParams>;
using BlsFp = Fe<BlsFpParams>;
using BlsFr = Fe<BlsFrParams>;

}  // namespace grape
