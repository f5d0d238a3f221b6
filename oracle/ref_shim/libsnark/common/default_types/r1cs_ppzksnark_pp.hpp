// Stand-in for the one libsnark/libff header the reference includes (include/ec_operation.cuh:5).
// TEST INFRASTRUCTURE ONLY: it lets the reference's own, unmodified sources compile where libsnark
// (fetched from the network by the reference's install.sh, unpinned) is not available.  It provides
// exactly the surface the reference uses: the scalar field `Fp_type` (memcpy-compatible with the
// device fr_t: four little-endian 64-bit words, Montgomery form), the group `libff::G1<ppT>`
// (memcpy-compatible with jacob_t: X|Y|Z), and `init_public_params()`.  The arithmetic is the C
// oracle's (oracle/grape_oracle.c); random_element() draws from a seedable SplitMix64 stream
// (ref_shim_seed) instead of libff's RNG so that runs are reproducible.
#pragma once
#include <cstdint>
#include <cstring>

extern "C" {
void oracle_fr_add(const void* a, const void* b, void* out);
void oracle_fr_sub(const void* a, const void* b, void* out);
void oracle_fr_mul(const void* a, const void* b, void* out);
void oracle_fr_inv(const void* a, void* out);
void oracle_fr_from_i64(int64_t v, void* out);
uint64_t oracle_rng_init(uint64_t seed, uint64_t tag);
void oracle_rng_fr(uint64_t* state, void* out);
void oracle_g1_add(const void* a, const void* b, void* out);
void oracle_g1_mul(const void* scalar, const void* p, void* out);
int oracle_g1_eq(const void* a, const void* b);
void oracle_g1_generator(void* out);
}

namespace ref_shim {
inline uint64_t& rng_state() {
  static uint64_t s = oracle_rng_init(0, 0);
  return s;
}
}  // namespace ref_shim
inline void ref_shim_seed(uint64_t seed) { ref_shim::rng_state() = oracle_rng_init(seed, 0); }

namespace libff {

struct ShimFr {
  uint64_t w[4];
  ShimFr() : w{0, 0, 0, 0} {}
  ShimFr(long v) { oracle_fr_from_i64((int64_t)v, w); }
  static ShimFr zero() { return ShimFr(); }
  static ShimFr one() { return ShimFr(1L); }
  static ShimFr random_element() {
    ShimFr r;
    oracle_rng_fr(&ref_shim::rng_state(), r.w);
    return r;
  }
  ShimFr operator+(const ShimFr& o) const { ShimFr r; oracle_fr_add(w, o.w, r.w); return r; }
  ShimFr operator-(const ShimFr& o) const { ShimFr r; oracle_fr_sub(w, o.w, r.w); return r; }
  ShimFr operator*(const ShimFr& o) const { ShimFr r; oracle_fr_mul(w, o.w, r.w); return r; }
  ShimFr operator-() const { ShimFr z, r; oracle_fr_sub(z.w, w, r.w); return r; }
  ShimFr& operator+=(const ShimFr& o) { oracle_fr_add(w, o.w, w); return *this; }
  ShimFr& operator-=(const ShimFr& o) { oracle_fr_sub(w, o.w, w); return *this; }
  ShimFr& operator*=(const ShimFr& o) { oracle_fr_mul(w, o.w, w); return *this; }
  ShimFr invert() const { ShimFr r; oracle_fr_inv(w, r.w); return r; }
  bool operator==(const ShimFr& o) const { return !std::memcmp(w, o.w, 32); }
  bool operator!=(const ShimFr& o) const { return !(*this == o); }
};

struct ShimG1 {
  uint64_t X[4], Y[4], Z[4];
  ShimG1() { std::memset(this, 0, sizeof(*this)); X[0] = Y[0] = 1; }  // Z = 0: infinity
  static ShimG1 zero() { return ShimG1(); }
  static ShimG1 random_element() {
    ShimG1 g, r;
    oracle_g1_generator(&g);
    ShimFr k = ShimFr::random_element();
    oracle_g1_mul(k.w, &g, &r);
    return r;
  }
  ShimG1 operator+(const ShimG1& o) const { ShimG1 r; oracle_g1_add(this, &o, &r); return r; }
  bool operator==(const ShimG1& o) const { return oracle_g1_eq(this, &o) != 0; }
};
inline ShimG1 operator*(const ShimFr& k, const ShimG1& p) { ShimG1 r; oracle_g1_mul(k.w, &p, &r); return r; }

template <class ppT>
using G1 = ShimG1;

}  // namespace libff

namespace libsnark {
struct default_r1cs_ppzksnark_pp {
  typedef libff::ShimFr Fp_type;
  static void init_public_params() {}
};
}  // namespace libsnark
