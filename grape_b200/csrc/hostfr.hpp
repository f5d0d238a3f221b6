// Host-side BN254 scalar-field arithmetic and the seedable random stream of the library.
//
// The reference does its small host-side algebra (round polynomials, claim updates) with libff's
// Fr and draws prover randomness from libff's RNG; this header is what stands in for both.  HostFr
// has the byte layout the reference relies on when it memcpy's between libff::Fr and device fr_t
// (src/fr-tensor.cu:214,366,437): four little-endian 64-bit words of value * 2^256 mod r.
#pragma once
#include <cstdint>
#include <cstring>

namespace grape {

struct HostFr {
  uint64_t w[4];
  bool operator==(const HostFr& o) const { return !std::memcmp(w, o.w, 32); }
  bool operator!=(const HostFr& o) const { return !(*this == o); }
};

namespace hostfr_detail {
static const uint64_t MOD[4] = {0x43e1f593f0000001ull, 0x2833e84879b97091ull, 0xb85045b68181585dull,
                                0x30644e72e131a029ull};
static const uint64_t R2[4] = {0x1bb8e645ae216da7ull, 0x53fe3ab1e35c59e3ull, 0x8c49833d53bb8085ull,
                               0x0216d0b17f4e44a5ull};
static const uint64_t ONE[4] = {0xac96341c4ffffffbull, 0x36fc76959f60cd29ull, 0x666ea36f7879462eull,
                                0x0e0a77c19a07df2full};
static const uint64_t INV = 0xc2e1f593efffffffull;  // -r^-1 mod 2^64
typedef unsigned __int128 u128;

inline bool geq_mod(const uint64_t* a) {
  for (int i = 3; i >= 0; i--) {
    if (a[i] > MOD[i]) return true;
    if (a[i] < MOD[i]) return false;
  }
  return true;
}
inline void sub_mod(uint64_t* a) {
  u128 borrow = 0;
  for (int i = 0; i < 4; i++) {
    u128 d = (u128)a[i] - MOD[i] - borrow;
    a[i] = (uint64_t)d;
    borrow = (d >> 64) & 1;
  }
}
}  // namespace hostfr_detail

inline HostFr fr_zero() { return HostFr{{0, 0, 0, 0}}; }
inline HostFr fr_one() {
  using namespace hostfr_detail;
  return HostFr{{ONE[0], ONE[1], ONE[2], ONE[3]}};
}

inline HostFr fr_add(const HostFr& a, const HostFr& b) {
  using namespace hostfr_detail;
  HostFr r;
  u128 c = 0;
  for (int i = 0; i < 4; i++) {
    c += (u128)a.w[i] + b.w[i];
    r.w[i] = (uint64_t)c;
    c >>= 64;
  }
  if (geq_mod(r.w)) sub_mod(r.w);
  return r;
}

inline HostFr fr_neg(const HostFr& a) {
  using namespace hostfr_detail;
  if (!(a.w[0] | a.w[1] | a.w[2] | a.w[3])) return a;
  HostFr r;
  u128 borrow = 0;
  for (int i = 0; i < 4; i++) {
    u128 d = (u128)MOD[i] - a.w[i] - borrow;
    r.w[i] = (uint64_t)d;
    borrow = (d >> 64) & 1;
  }
  return r;
}

inline HostFr fr_sub(const HostFr& a, const HostFr& b) { return fr_add(a, fr_neg(b)); }

// Montgomery product (CIOS over 64-bit words).
inline HostFr fr_mul(const HostFr& a, const HostFr& b) {
  using namespace hostfr_detail;
  uint64_t t[6] = {0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 4; i++) {
    u128 c = 0;
    for (int j = 0; j < 4; j++) {
      c += (u128)a.w[j] * b.w[i] + t[j];
      t[j] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[4] = (uint64_t)c;
    t[5] = (uint64_t)(c >> 64);
    uint64_t m = t[0] * INV;
    c = (u128)m * MOD[0] + t[0];
    c >>= 64;
    for (int j = 1; j < 4; j++) {
      c += (u128)m * MOD[j] + t[j];
      t[j - 1] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[3] = (uint64_t)c;
    t[4] = t[5] + (uint64_t)(c >> 64);
  }
  HostFr r{{t[0], t[1], t[2], t[3]}};
  if (t[4] || geq_mod(r.w)) sub_mod(r.w);
  return r;
}

inline HostFr fr_from_raw(const uint64_t raw[4]) {  // standard-form integer < 2^256 -> Montgomery
  using namespace hostfr_detail;
  HostFr x{{raw[0], raw[1], raw[2], raw[3]}};
  return fr_mul(x, HostFr{{R2[0], R2[1], R2[2], R2[3]}});
}

inline HostFr fr_from_u64(uint64_t v) {
  uint64_t raw[4] = {v, 0, 0, 0};
  return fr_from_raw(raw);
}

inline HostFr fr_from_i64(int64_t v) {
  if (v >= 0) return fr_from_u64((uint64_t)v);
  return fr_neg(fr_from_u64((uint64_t)(-(v + 1)) + 1));
}

inline HostFr fr_pow(const HostFr& a, const uint64_t e[4]) {
  HostFr acc = fr_one();
  for (int i = 3; i >= 0; i--)
    for (int b = 63; b >= 0; b--) {
      acc = fr_mul(acc, acc);
      if ((e[i] >> b) & 1) acc = fr_mul(acc, a);
    }
  return acc;
}

inline HostFr fr_inv(const HostFr& a) {
  using namespace hostfr_detail;
  uint64_t e[4] = {MOD[0] - 2, MOD[1], MOD[2], MOD[3]};
  return fr_pow(a, e);
}

// eq(u, v) = uv + (1-u)(1-v)   (reference: Polynomial::eq, src/polynomial.cu:47-53)
inline HostFr fr_eq2(const HostFr& u, const HostFr& v) {
  HostFr uv = fr_mul(u, v);
  return fr_add(fr_sub(fr_add(uv, uv), fr_add(u, v)), fr_one());
}

// ---- SplitMix64 stream: the library's stand-in for libff's Fr::random_element() ----------------
inline uint64_t splitmix_init(uint64_t seed, uint64_t tag) {
  return seed * 0x9E3779B97F4A7C15ull + tag * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
}
inline uint64_t splitmix_next(uint64_t& state) {
  state += 0x9E3779B97F4A7C15ull;
  uint64_t z = state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
// 512 random bits (eight words, little-endian) reduced mod r: lo + hi * 2^256.
inline HostFr rng_next_fr(uint64_t& state) {
  using namespace hostfr_detail;
  uint64_t lo[4], hi[4];
  for (int i = 0; i < 4; i++) lo[i] = splitmix_next(state);
  for (int i = 0; i < 4; i++) hi[i] = splitmix_next(state);
  // Montgomery(lo) = lo*R ; Montgomery(hi*2^256) = hi*R*R = mont_mul(hi*R... ) computed as
  // fr_mul(fr_from_raw(hi), R2-as-Montgomery-of-R) = hi * R * R.
  HostFr a = fr_from_raw(lo);
  HostFr b = fr_from_raw(hi);
  HostFr r2{{R2[0], R2[1], R2[2], R2[3]}};  // R^2 mod r, i.e. the Montgomery form of R = 2^256
  return fr_add(a, fr_mul(b, r2));
}

}  // namespace grape
