// Host-side G1 arithmetic of BN254 for the C++ veneer: what the reference's drivers do with libff's
// alt_bn128_G1 on the host (the verifier block of test/HyraxTest.cu:88-125, host_partial_me<bn128> in
// include/ec_operation.cuh:37-55, `sum_ad * G` in src/Hyrax.cu:291).  Points are 96-byte Jacobian
// records X|Y|Z of Montgomery residues, the layout libff::G1 shares with the device jacob_t
// (src/ec_operation.cu:40); Z = 0 is the point at infinity.  Not on the proving hot path: nothing here
// is called by the provers, which do their group arithmetic on the GPU.
#include <cstdint>
#include <cstring>

#include "../../include/grape_b200.h"
#include "hostfr.hpp"

namespace {

using grape::HostFr;
typedef unsigned __int128 u128;

struct Fp {
  uint64_t w[4];
};
const uint64_t P_MOD[4] = {0x3c208c16d87cfd47ull, 0x97816a916871ca8dull, 0xb85045b68181585dull, 0x30644e72e131a029ull};
const uint64_t P_ONE[4] = {0xd35d438dc58f0d9dull, 0x0a78eb28f5c70b3dull, 0x666ea36f7879462cull, 0x0e0a77c19a07df2full};
const uint64_t P_INV = 0x87d20782e4866389ull;  // -p^-1 mod 2^64

inline bool is_zero(const Fp& a) { return !(a.w[0] | a.w[1] | a.w[2] | a.w[3]); }
inline bool geq_p(const uint64_t* a) {
  for (int i = 3; i >= 0; i--) {
    if (a[i] > P_MOD[i]) return true;
    if (a[i] < P_MOD[i]) return false;
  }
  return true;
}
inline void sub_p(uint64_t* a) {
  u128 borrow = 0;
  for (int i = 0; i < 4; i++) {
    u128 d = (u128)a[i] - P_MOD[i] - borrow;
    a[i] = (uint64_t)d;
    borrow = (d >> 64) & 1;
  }
}
inline Fp fp_add(const Fp& a, const Fp& b) {
  Fp r;
  u128 c = 0;
  for (int i = 0; i < 4; i++) {
    c += (u128)a.w[i] + b.w[i];
    r.w[i] = (uint64_t)c;
    c >>= 64;
  }
  if (geq_p(r.w)) sub_p(r.w);
  return r;
}
inline Fp fp_neg(const Fp& a) {
  if (is_zero(a)) return a;
  Fp r;
  u128 borrow = 0;
  for (int i = 0; i < 4; i++) {
    u128 d = (u128)P_MOD[i] - a.w[i] - borrow;
    r.w[i] = (uint64_t)d;
    borrow = (d >> 64) & 1;
  }
  return r;
}
inline Fp fp_sub(const Fp& a, const Fp& b) { return fp_add(a, fp_neg(b)); }
inline Fp fp_dbl(const Fp& a) { return fp_add(a, a); }
inline Fp fp_mul(const Fp& a, const Fp& b) {  // Montgomery product, CIOS over 64-bit words
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
    uint64_t m = t[0] * P_INV;
    c = (u128)m * P_MOD[0] + t[0];
    c >>= 64;
    for (int j = 1; j < 4; j++) {
      c += (u128)m * P_MOD[j] + t[j];
      t[j - 1] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[3] = (uint64_t)c;
    t[4] = t[5] + (uint64_t)(c >> 64);
  }
  Fp r{{t[0], t[1], t[2], t[3]}};
  if (t[4] || geq_p(r.w)) sub_p(r.w);
  return r;
}
inline Fp fp_sqr(const Fp& a) { return fp_mul(a, a); }
inline Fp fp_one() { return Fp{{P_ONE[0], P_ONE[1], P_ONE[2], P_ONE[3]}}; }
inline Fp fp_inv(const Fp& a) {  // a^(p-2)
  uint64_t e[4] = {P_MOD[0] - 2, P_MOD[1], P_MOD[2], P_MOD[3]};
  Fp acc = fp_one();
  for (int i = 3; i >= 0; i--)
    for (int b = 63; b >= 0; b--) {
      acc = fp_sqr(acc);
      if ((e[i] >> b) & 1) acc = fp_mul(acc, a);
    }
  return acc;
}

struct Jac {
  Fp x, y, z;
};
inline Jac jac_inf() { return Jac{fp_one(), fp_one(), Fp{{0, 0, 0, 0}}}; }
inline Jac jac_dbl(const Jac& p) {  // a = 0 short Weierstrass
  if (is_zero(p.z) || is_zero(p.y)) return jac_inf();
  Fp A = fp_sqr(p.x), B = fp_sqr(p.y), C = fp_sqr(B);
  Fp D = fp_dbl(fp_sub(fp_sub(fp_sqr(fp_add(p.x, B)), A), C));
  Fp E = fp_add(fp_dbl(A), A), F = fp_sqr(E);
  Jac r;
  r.x = fp_sub(F, fp_dbl(D));
  Fp C8 = fp_dbl(fp_dbl(fp_dbl(C)));
  r.y = fp_sub(fp_mul(E, fp_sub(D, r.x)), C8);
  r.z = fp_dbl(fp_mul(p.y, p.z));
  return r;
}
inline Jac jac_add(const Jac& p, const Jac& q) {
  if (is_zero(p.z)) return q;
  if (is_zero(q.z)) return p;
  Fp Z1Z1 = fp_sqr(p.z), Z2Z2 = fp_sqr(q.z);
  Fp U1 = fp_mul(p.x, Z2Z2), U2 = fp_mul(q.x, Z1Z1);
  Fp S1 = fp_mul(fp_mul(p.y, q.z), Z2Z2), S2 = fp_mul(fp_mul(q.y, p.z), Z1Z1);
  Fp H = fp_sub(U2, U1), Rr = fp_sub(S2, S1);
  if (is_zero(H)) return is_zero(Rr) ? jac_dbl(p) : jac_inf();
  Fp HH = fp_sqr(H), HHH = fp_mul(H, HH), V = fp_mul(U1, HH);
  Jac r;
  r.x = fp_sub(fp_sub(fp_sqr(Rr), HHH), fp_dbl(V));
  r.y = fp_sub(fp_mul(Rr, fp_sub(V, r.x)), fp_mul(S1, HHH));
  r.z = fp_mul(fp_mul(p.z, q.z), H);
  return r;
}
inline Jac jac_normalise(const Jac& p) {
  if (is_zero(p.z)) return jac_inf();
  Fp zi = fp_inv(p.z), zi2 = fp_sqr(zi);
  return Jac{fp_mul(p.x, zi2), fp_mul(p.y, fp_mul(zi2, zi)), fp_one()};
}
inline Jac jac_scalar_mul(const HostFr& k_mont, const Jac& p) {
  const HostFr raw_one{{1, 0, 0, 0}};
  const HostFr k = grape::fr_mul(k_mont, raw_one);  // leave Montgomery form
  Jac acc = jac_inf();
  for (int i = 3; i >= 0; i--)
    for (int b = 63; b >= 0; b--) {
      acc = jac_dbl(acc);
      if ((k.w[i] >> b) & 1) acc = jac_add(acc, p);
    }
  return acc;
}
inline Jac load(const void* p) {
  Jac j;
  std::memcpy(&j, p, 96);
  return j;
}
}  // namespace

extern "C" void grape_hg1_add(const void* a, const void* b, void* out) {
  Jac r = jac_add(load(a), load(b));
  std::memcpy(out, &r, 96);
}
extern "C" void grape_hg1_scalar_mul(const void* h_fr, const void* p, void* out) {
  HostFr k;
  std::memcpy(&k, h_fr, 32);
  Jac r = jac_scalar_mul(k, load(p));
  std::memcpy(out, &r, 96);
}
extern "C" void grape_hg1_neg(const void* a, void* out) {
  Jac r = load(a);
  r.y = fp_neg(r.y);
  std::memcpy(out, &r, 96);
}
extern "C" void grape_hg1_normalise(const void* a, void* out) {
  Jac r = jac_normalise(load(a));
  std::memcpy(out, &r, 96);
}
extern "C" int grape_hg1_equal(const void* a, const void* b) {
  Jac p = load(a), q = load(b);
  const bool pi = is_zero(p.z), qi = is_zero(q.z);
  if (pi || qi) return pi && qi;
  Fp Z1Z1 = fp_sqr(p.z), Z2Z2 = fp_sqr(q.z);
  if (std::memcmp(fp_mul(p.x, Z2Z2).w, fp_mul(q.x, Z1Z1).w, 32)) return 0;
  return !std::memcmp(fp_mul(fp_mul(p.y, q.z), Z2Z2).w, fp_mul(fp_mul(q.y, p.z), Z1Z1).w, 32);
}
