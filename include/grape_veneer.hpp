// C++ veneer over the C ABI (grape_b200.h) that re-creates the host API of the reference for the
// proving path: the same class and function names, argument meaning and error behaviour
// (std::runtime_error), so that drivers written against the reference's headers
// (include/fr-tensor.cuh, Hyrax.cuh, ec_operation.cuh, prove.cuh, tlookup.cuh) compile against
// this header instead.  Header-only; link with libgrape_b200.so.  Differences are noted where
// they exist: the table handed to Hyrax may be the reference's points.bin layout or the B200
// layout, random draws come from a seedable stream, and tensors passed to the provers are
// consumed rather than folded to a specific state.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "grape_b200.h"

typedef unsigned int uint;

namespace grape_veneer {

inline grape_ctx*& ctx_slot() {
  static grape_ctx* c = nullptr;
  return c;
}
// The implicit device of the reference: one process-wide context on device 0 (or GRAPE_DEVICE).
inline grape_ctx* ctx() {
  grape_ctx*& c = ctx_slot();
  if (!c) {
    int dev = 0;
    if (const char* e = std::getenv("GRAPE_DEVICE")) dev = std::atoi(e);
    if (grape_ctx_create(dev, &c) != GRAPE_OK) throw std::runtime_error("grape_b200: no usable CUDA device");
  }
  return c;
}
inline void check(int rc) {
  if (rc != GRAPE_OK) throw std::runtime_error(grape_ctx_error(ctx_slot()));
}
inline void* dev_alloc(size_t bytes) {
  void* p = nullptr;
  check(grape_dev_alloc(ctx(), bytes ? bytes : 1, &p));
  return p;
}

}  // namespace grape_veneer

// ---- Fr: the host scalar (libff's alt_bn128 Fr in the reference, include/ec_operation.cuh:11-14) ----
struct Fr {
  uint64_t w[4];
  Fr() : w{0, 0, 0, 0} {}
  Fr(long v) { grape_hfr_from_i64((int64_t)v, w); }
  static Fr zero() { return Fr(); }
  static Fr one() { return Fr(1L); }
  static Fr random_element() {
    Fr r;
    grape_veneer::check(grape_rng_fr(grape_veneer::ctx(), r.w, 1));
    return r;
  }
  Fr operator+(const Fr& o) const { Fr r; grape_hfr_add(w, o.w, r.w); return r; }
  Fr operator-(const Fr& o) const { Fr r; grape_hfr_sub(w, o.w, r.w); return r; }
  Fr operator*(const Fr& o) const { Fr r; grape_hfr_mul(w, o.w, r.w); return r; }
  Fr operator-() const { Fr z, r; grape_hfr_sub(z.w, w, r.w); return r; }
  Fr& operator+=(const Fr& o) { grape_hfr_add(w, o.w, w); return *this; }
  Fr& operator-=(const Fr& o) { grape_hfr_sub(w, o.w, w); return *this; }
  Fr& operator*=(const Fr& o) { grape_hfr_mul(w, o.w, w); return *this; }
  Fr invert() const { Fr r; grape_hfr_inv(w, r.w); return r; }
  bool operator==(const Fr& o) const { return !std::memcmp(w, o.w, 32); }
  bool operator!=(const Fr& o) const { return !(*this == o); }
};

// Device records, byte-compatible with the reference's fr_t / affine_t / jacob_t.
struct fr_t { uint32_t v[8]; };
struct affine_t { uint32_t v[16]; };
struct jacob_t { uint32_t v[24]; };
// Host G1 point (libff G1 in the reference); outputs of this library are normalised, so equal
// group elements have equal bytes.
struct bn128 {
  uint32_t v[24];
  bool operator==(const bn128& o) const { return !std::memcmp(v, o.v, 96); }
};

inline uint Log2(uint num) {  // ceil(log2), src/ioutils.cu:173-190
  if (num == 0) return 0;
  num--;
  uint r = 0;
  while (num > 0) { num >>= 1; r++; }
  return r;
}

inline std::vector<Fr> random_vec(uint len) {  // src/ec_operation.cu:51-57
  std::vector<Fr> out(len);
  for (auto& x : out) x = Fr::random_element();
  return out;
}
inline void generate_random_eval_points(size_t data_size, std::vector<Fr>& eval_point) {  // :59-71
  eval_point.resize(Log2((uint)data_size));
  for (auto& x : eval_point) x = Fr::random_element();
}
inline void ReassembleVectors(std::vector<Fr>& first, std::vector<Fr>& second, size_t first_size, size_t same_size,
                              size_t last_size) {  // src/ec_operation.cu:74-122
  std::vector<Fr> r1, r2;
  r1.insert(r1.end(), second.begin(), second.begin() + same_size);
  r1.insert(r1.end(), first.begin() + last_size, first.begin() + last_size + first_size);
  r1.insert(r1.end(), second.begin() + same_size, second.end());
  r2.insert(r2.end(), second.begin(), second.begin() + same_size);
  r2.insert(r2.end(), first.begin(), first.begin() + last_size);
  r2.insert(r2.end(), second.begin() + same_size, second.end());
  first = r1;
  second = r2;
}

// ---- FrTensor (include/fr-tensor.cuh:36-76) ---------------------------------------------------
class FrTensor {
 public:
  fr_t* gpu_data;
  uint size;

  explicit FrTensor(uint size_) : gpu_data((fr_t*)grape_veneer::dev_alloc((size_t)size_ * 32)), size(size_), cap_(size_) {}
  FrTensor(const FrTensor& t) : gpu_data((fr_t*)grape_veneer::dev_alloc((size_t)t.size * 32)), size(t.size), cap_(t.size) {
    grape_veneer::check(grape_d2d(grape_veneer::ctx(), gpu_data, t.gpu_data, (size_t)size * 32));
  }
  FrTensor(uint size_, int* device_ints) : FrTensor(size_) {
    grape_veneer::check(grape_fr_from_i32(grape_veneer::ctx(), device_ints, gpu_data, size));
  }
  ~FrTensor() {
    if (gpu_data) grape_dev_free(grape_veneer::ctx(), gpu_data);
  }
  // copies min(size) elements without reallocating, like the reference (src/fr-tensor.cu:322-328)
  FrTensor& operator=(const FrTensor& x) {
    uint n = size < x.size ? size : x.size;
    grape_veneer::check(grape_d2d(grape_veneer::ctx(), gpu_data, x.gpu_data, (size_t)n * 32));
    return *this;
  }
  void set_size(uint sz) {
    if (sz > cap_) throw std::runtime_error("FrTensor::set_size beyond the allocation");
    size = sz;
  }
  void get_data(uint sz, int* device_ints) {
    set_size(sz);
    grape_veneer::check(grape_fr_from_i32(grape_veneer::ctx(), device_ints, gpu_data, sz));
  }
  void get_data(uint sz, uint* device_uints) {
    set_size(sz);
    grape_veneer::check(grape_fr_from_u32(grape_veneer::ctx(), device_uints, gpu_data, sz));
  }
  // fold of axis c of the [N/(c*gap)][c][gap] view with challenges x[id..], result compacted to the front
  void partial_eval(uint N, fr_t* x, uint c, uint id, uint gap) {
    FrTensor tmp(N / c ? N / c : 1);
    grape_veneer::check(grape_fr_fold(grape_veneer::ctx(), gpu_data, N, x + id, c, gap, tmp.gpu_data));
    grape_veneer::check(grape_d2d(grape_veneer::ctx(), gpu_data, tmp.gpu_data, (size_t)(N / c) * 32));
    grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
  }
  // full multilinear evaluation (src/fr-tensor.cu:346-369); tensors shorter than 2^|u| are taken to
  // have rows of 11008 padded to 16384, as the reference hard-codes
  Fr operator()(const std::vector<Fr>& u) {
    grape_ctx* c = grape_veneer::ctx();
    fr_t* d_u = (fr_t*)grape_veneer::dev_alloc(u.size() * 32 + 32);
    grape_veneer::check(grape_h2d(c, d_u, u.data(), u.size() * 32));
    if (size < (1u << u.size())) {
      partial_eval(size, d_u, size / 11008, Log2(11008), 11008);
      partial_eval(11008, d_u, 11008, 0, 1);
    } else {
      partial_eval(size, d_u, size, 0, 1);
    }
    Fr ret;
    grape_veneer::check(grape_d2h(c, ret.w, gpu_data, 32));
    grape_dev_free(c, d_u);
    return ret;
  }
  Fr operator()(uint idx) const {
    Fr out;
    grape_veneer::check(grape_d2h(grape_veneer::ctx(), out.w, gpu_data + idx, 32));
    return out;
  }
  void add_with_size(uint sz, const FrTensor& t) { grape_veneer::check(grape_fr_add(grape_veneer::ctx(), gpu_data, t.gpu_data, gpu_data, sz)); }
  void mul_with_size(uint sz, const FrTensor& t) { grape_veneer::check(grape_fr_mul(grape_veneer::ctx(), gpu_data, t.gpu_data, gpu_data, sz)); }
  void mul_with_size(uint sz, fr_t* x) { grape_veneer::check(grape_fr_scale(grape_veneer::ctx(), gpu_data, x, gpu_data, sz)); }
  void mul_with_size(uint sz, Fr& x) { scalar_op(sz, x, true); }
  void inverse() { grape_veneer::check(grape_fr_inverse(grape_veneer::ctx(), gpu_data, nullptr, gpu_data, size)); }
  void from() { grape_veneer::check(grape_fr_from_mont(grape_veneer::ctx(), gpu_data, size)); }
  void to() { grape_veneer::check(grape_fr_to_mont(grape_veneer::ctx(), gpu_data, size)); }
  Fr sum(uint sz) {
    grape_ctx* c = grape_veneer::ctx();
    void* d = grape_veneer::dev_alloc(32);
    grape_veneer::check(grape_fr_sum(c, gpu_data, sz, d));
    Fr out;
    grape_veneer::check(grape_d2h(c, out.w, d, 32));
    grape_dev_free(c, d);
    return out;
  }
  FrTensor sum(uint sz, uint N) {  // every element replaced by its row sum (src/fr-tensor.cu:442-449)
    if (sz % N) throw std::runtime_error("FrTensor::sum: size is not a multiple of the row length");
    FrTensor out(sz);
    grape_veneer::check(grape_fr_rowsum(grape_veneer::ctx(), gpu_data, out.gpu_data, sz / N, N));
    return out;
  }
  void pad(FrTensor& tmp, uint N, uint pad_N, uint pad_size, const Fr& pad_val) {  // src/fr-tensor.cu:458-466
    if (N == pad_N) return;
    grape_ctx* c = grape_veneer::ctx();
    void* d = grape_veneer::dev_alloc(32);
    grape_veneer::check(grape_h2d(c, d, pad_val.w, 32));
    grape_veneer::check(grape_fr_pad(c, gpu_data, tmp.gpu_data, N, pad_N, pad_size, d));
    set_size(pad_size);
    grape_veneer::check(grape_d2d(c, gpu_data, tmp.gpu_data, (size_t)pad_size * 32));
    grape_dev_free(c, d);
  }
  FrTensor& operator+=(const FrTensor& t) { same(t); add_with_size(size, t); return *this; }
  FrTensor& operator-=(const FrTensor& t) { same(t); grape_veneer::check(grape_fr_sub(grape_veneer::ctx(), gpu_data, t.gpu_data, gpu_data, size)); return *this; }
  FrTensor& operator*=(const FrTensor& t) { same(t); mul_with_size(size, t); return *this; }
  FrTensor& operator*=(fr_t* x) { mul_with_size(size, x); return *this; }
  FrTensor& operator*=(Fr& x) { scalar_op(size, x, true); return *this; }
  FrTensor& operator*=(const uint x) { Fr f((long)x); scalar_op(size, f, true); return *this; }
  FrTensor& operator+=(const int x) { Fr f((long)x); scalar_op(size, f, false); return *this; }
  static FrTensor random(uint size) {
    std::vector<Fr> tmp = random_vec(size);
    FrTensor out(size);
    grape_veneer::check(grape_h2d(grape_veneer::ctx(), out.gpu_data, tmp.data(), (size_t)size * 32));
    grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
    return out;
  }

 private:
  uint cap_;
  void same(const FrTensor& t) const {
    if (size != t.size) throw std::runtime_error("Incompatible dimensions");
  }
  void scalar_op(uint sz, const Fr& x, bool mul) {
    grape_ctx* c = grape_veneer::ctx();
    void* d = grape_veneer::dev_alloc(32);
    grape_veneer::check(grape_h2d(c, d, x.w, 32));
    grape_veneer::check(mul ? grape_fr_scale(c, gpu_data, d, gpu_data, sz) : grape_fr_add_scalar(c, gpu_data, d, gpu_data, sz));
    grape_dev_free(c, d);
  }
};

inline void Fr_partial_me(uint N, FrTensor& t, fr_t* x, uint id, uint cur_dim, uint window_size) {
  // the reference leaves the result strided in place; callers only ever read it after the
  // compaction done by partial_eval, which is what this forwards to
  t.partial_eval(N, x, cur_dim, id, window_size);
}

inline void pad_int(int** int_data, uint N, uint pad_N, uint pad_size) {  // src/fr-tensor.cu:190-200
  if (N == pad_N) return;
  grape_ctx* c = grape_veneer::ctx();
  int* fresh = (int*)grape_veneer::dev_alloc((size_t)pad_size * 4);
  grape_veneer::check(grape_pad_i32(c, *int_data, fresh, N, pad_N, pad_size));
  grape_dev_free(c, *int_data);
  *int_data = fresh;
}

// ---- Hyrax (include/Hyrax.cuh:57-86) -----------------------------------------------------------
class Hyrax_proof {
 public:
  size_t z_size;
  Fr result;
  Fr* z;
  bn128 commit_d;
  bn128 commit_ad;
  Hyrax_proof(Fr result_, size_t z_len, bn128 commit_d_, bn128 commit_ad_)
      : z_size(z_len), result(result_), z(new Fr[z_len]), commit_d(commit_d_), commit_ad(commit_ad_) {}
  ~Hyrax_proof() { delete[] z; }
  Hyrax_proof(const Hyrax_proof& o) : z_size(o.z_size), result(o.result), z(new Fr[o.z_size]), commit_d(o.commit_d), commit_ad(o.commit_ad) {
    for (size_t i = 0; i < z_size; i++) z[i] = o.z[i];
  }
  Hyrax_proof& operator=(const Hyrax_proof& o) {
    if (this != &o) {
      delete[] z;
      z_size = o.z_size; result = o.result; commit_d = o.commit_d; commit_ad = o.commit_ad;
      z = new Fr[z_size];
      for (size_t i = 0; i < z_size; i++) z[i] = o.z[i];
    }
    return *this;
  }
};

class Hyrax {
 public:
  uint com_scale;
  uint layer_num;
  uint npoints;  // generators per row capacity = npoints_ * com_scale
  bn128 G;
  affine_t* g_affine;
  grape_table* table;

  // g: the reference's table layout (256 rows of npoints_*16 affine points, row w = w * G_i)
  Hyrax(uint layer_num_, uint npoints_, affine_t* g, bn128& G_)
      : com_scale(16), layer_num(layer_num_), npoints(npoints_ * 16), G(G_), g_affine(g), table(nullptr) {
    grape_veneer::check(grape_table_from_reference(grape_veneer::ctx(), g, npoints, &table));
  }
  // B200 layout built by grape_table_create (signed digits, 8- or 16-bit windows)
  Hyrax(uint layer_num_, uint npoints_, grape_table* t, bn128& G_)
      : com_scale(16), layer_num(layer_num_), npoints(npoints_ * 16), G(G_), g_affine(nullptr), table(t), borrowed_(true) {}
  ~Hyrax() {
    if (table && !borrowed_) grape_table_destroy(table);
  }
  jacob_t* commit(int* tensor, uint size, uint N) {
    shape(size, N);
    jacob_t* out = (jacob_t*)grape_veneer::dev_alloc((size_t)(size / (N * com_scale)) * 96);
    grape_veneer::check(grape_commit_i32(grape_veneer::ctx(), table, tensor, size, N * com_scale, 32, out));
    grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
    return out;  // caller frees (grape_dev_free / cudaFree), as with the reference
  }
  jacob_t* commit(FrTensor& tensor, uint size, uint N) {
    shape(size, N);
    jacob_t* out = (jacob_t*)grape_veneer::dev_alloc((size_t)(size / (N * com_scale)) * 96);
    grape_veneer::check(grape_commit_fr(grape_veneer::ctx(), table, tensor.gpu_data, size, N * com_scale, out));
    grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
    return out;
  }
  Hyrax_proof open(FrTensor& tensor, const std::vector<Fr> eval_point_, Fr c, uint size, uint N) {
    if (size / N / com_scale < layer_num) throw std::runtime_error("Size too small: size < N * com_scale * layer_num");
    const uint new_N = (1u << Log2(N)) * com_scale;
    Hyrax_proof proof(Fr::zero(), new_N, G, G);
    grape_veneer::check(grape_hyrax_open(grape_veneer::ctx(), table, tensor.gpu_data, size, N, layer_num, eval_point_.data(),
                                         (uint32_t)eval_point_.size(), c.w, G.v, proof.result.w, proof.z, proof.commit_d.v,
                                         proof.commit_ad.v));
    return proof;
  }

 private:
  bool borrowed_ = false;
  void shape(uint size, uint N) const {
    if (size / N / com_scale < layer_num) throw std::runtime_error("Size too small: size < N * com_scale * layer_num");
    if (N != (1u << Log2(N))) throw std::runtime_error("N must be a power of 2");
  }
};

inline void single_commit(fr_t* d, grape_table* table, jacob_t* com, uint N) {  // src/Hyrax.cu:176-185
  grape_veneer::check(grape_commit_fr(grape_veneer::ctx(), table, d, N, N, com));
  grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
}

// ---- provers (include/prove.cuh:36-55) ---------------------------------------------------------
inline std::pair<Fr, Fr> prove_matmul(FrTensor& A, FrTensor& B, int L, int N, int M, int K, const std::vector<Fr> u,
                                      const std::vector<Fr> v, Fr& claim) {
  Fr out[2];
  grape_veneer::check(grape_prove_matmul(grape_veneer::ctx(), A.gpu_data, B.gpu_data, L, N, M, K, u.data(), (uint32_t)u.size(),
                                         v.data(), (uint32_t)v.size(), claim.w, out, nullptr, 0, nullptr));
  return {out[0], out[1]};
}
inline std::pair<Fr, Fr> prove_eleMul(FrTensor& A, FrTensor& B, int L, int M, int N, const std::vector<Fr> u,
                                      const std::vector<Fr> v, Fr& claim) {
  Fr out[2];
  grape_veneer::check(grape_prove_elemul(grape_veneer::ctx(), A.gpu_data, B.gpu_data, L, M, N, u.data(), (uint32_t)u.size(),
                                         v.data(), (uint32_t)v.size(), claim.w, out, nullptr, 0, nullptr));
  return {out[0], out[1]};
}
inline Fr combine_claims(FrTensor& X, const std::vector<Fr>& claims, const std::vector<std::vector<Fr>>& u,
                         const std::vector<Fr>& v, const uint size) {
  std::vector<Fr> flat;
  for (auto& uj : u) {
    if (uj.size() != v.size()) throw std::runtime_error("combine_claims: challenge vectors differ in length");
    flat.insert(flat.end(), uj.begin(), uj.end());
  }
  Fr out;
  grape_veneer::check(grape_combine_claims(grape_veneer::ctx(), X.gpu_data, size, claims.data(), (uint32_t)claims.size(),
                                           flat.data(), v.data(), (uint32_t)v.size(), out.w, nullptr, 0, nullptr));
  return out;
}

// ---- lookup argument (include/tlookup.cuh:37-79) -----------------------------------------------
class tLookupRange {
 public:
  Fr alpha, beta;
  const int low;
  grape_lookup* handle;
  tLookupRange(int low_, uint len) : low(low_), handle(nullptr) {
    grape_veneer::check(grape_lookup_range_create(grape_veneer::ctx(), low_, len, &handle));
    grape_lookup_params(handle, alpha.w, beta.w, nullptr, nullptr);
  }
  ~tLookupRange() { grape_lookup_destroy(handle); }
  tLookupRange(const tLookupRange&) = delete;
  // S and A as in the reference: S the queries (consumed), A scratch of the padded size
  Fr prove(FrTensor& S, FrTensor& A, const std::vector<Fr>& v, Hyrax& hyrax, uint msm_size, double& commit_time) {
    (void)commit_time;
    Fr out;
    grape_veneer::check(grape_lookup_prove_range(grape_veneer::ctx(), handle, S.gpu_data, S.size, A.gpu_data, v.data(),
                                                 (uint32_t)v.size(), 11008, 16384, hyrax.table, msm_size, nullptr, nullptr,
                                                 out.w, nullptr, 0, nullptr));
    return out;
  }
};

class tLookupRangeMapping {
 public:
  Fr alpha, beta, r;
  int low;
  grape_lookup* handle;
  // d_map: the int32 table f in device memory (the reference reads it from a file, src/tlookup.cu:355-358)
  tLookupRangeMapping(const int low_, const uint len, const int* d_map) : low(low_), handle(nullptr) {
    grape_veneer::check(grape_lookup_mapping_create(grape_veneer::ctx(), low_, len, d_map, &handle));
    grape_lookup_params(handle, alpha.w, beta.w, r.w, nullptr);
  }
  ~tLookupRangeMapping() { grape_lookup_destroy(handle); }
  tLookupRangeMapping(const tLookupRangeMapping&) = delete;
  Fr prove(FrTensor& S_in, FrTensor& S_out, FrTensor& A, const std::vector<Fr>& v, Hyrax& hyrax, uint msm_size,
           double& commit_time) {
    (void)commit_time;
    FrTensor work(1u << Log2(S_in.size));
    Fr out;
    grape_veneer::check(grape_lookup_prove_mapping(grape_veneer::ctx(), handle, S_in.gpu_data, S_out.gpu_data, S_in.size,
                                                   work.gpu_data, A.gpu_data, v.data(), (uint32_t)v.size(), 11008, 16384,
                                                   hyrax.table, msm_size, nullptr, nullptr, out.w, nullptr, 0, nullptr));
    return out;
  }
};
