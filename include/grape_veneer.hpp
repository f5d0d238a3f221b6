// C++ veneer over the C ABI (grape_b200.h) that re-creates the host API of the reference for the
// proving path: the same class and function names, argument meaning and error behaviour
// (std::runtime_error), so that drivers written against the reference's headers
// (include/fr-tensor.cuh, Hyrax.cuh, ec_operation.cuh, prove.cuh, tlookup.cuh) compile against
// this header instead.  Header-only; link with libgrape_b200.so.  Differences are noted where
// they exist: the table handed to Hyrax may be the reference's points.bin layout or the B200
// layout, random draws come from a seedable stream, and tensors passed to the provers are
// consumed rather than folded to a specific state.
#pragma once
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <limits>
#include <mutex>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "grape_b200.h"

typedef unsigned int uint;
typedef unsigned long ulong;

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
  static Fr random_element() {  // the reference's drivers draw inside OpenMP loops (test/HyraxTest.cu:73-76)
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
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
// Host G1 point (libff's alt_bn128_G1 in the reference, include/ec_operation.cuh:11-14): a 96-byte
// Jacobian record with the group operations the drivers use on the host.  Equality is equality of
// group elements, whatever the Z coordinates.
struct bn128 {
  uint32_t v[24];
  bn128() { std::memset(v, 0, 96); }  // the point at infinity (any record with Z = 0)
  static bn128 zero() { return bn128(); }
  static bn128 one() {  // the generator (1, 2), Z = 1
    static const uint32_t fp_one[8] = {0xc58f0d9du, 0xd35d438du, 0xf5c70b3du, 0x0a78eb28u,
                                       0x7879462cu, 0x666ea36fu, 0x9a07df2fu, 0x0e0a77c1u};  // 2^256 mod p
    static const uint32_t fp_two[8] = {0x8b1e1b3au, 0xa6ba871bu, 0xeb8e167bu, 0x14f1d651u,
                                       0xf0f28c58u, 0xccdd46deu, 0x340fbe5eu, 0x1c14ef83u};  // 2 * 2^256 mod p
    bn128 r;
    std::memcpy(r.v, fp_one, 32);
    std::memcpy(r.v + 8, fp_two, 32);
    std::memcpy(r.v + 16, fp_one, 32);
    return r;
  }
  static bn128 random_element() { return Fr::random_element() * one(); }
  bn128 operator+(const bn128& o) const { bn128 r; grape_hg1_add(v, o.v, r.v); return r; }
  bn128 operator-() const { bn128 r; grape_hg1_neg(v, r.v); return r; }
  bn128 operator-(const bn128& o) const { return *this + (-o); }
  friend bn128 operator*(const Fr& k, const bn128& p) { bn128 r; grape_hg1_scalar_mul(k.w, p.v, r.v); return r; }
  bool operator==(const bn128& o) const { return grape_hg1_equal(v, o.v) != 0; }
  bool operator!=(const bn128& o) const { return !(*this == o); }

};

// The reference's drivers open with `using namespace libsnark;` and `ppT::init_public_params();`
// (include/ec_operation.cuh:9-14): nothing to set up here.
namespace libsnark {}
namespace libff {}
struct ppT {
  static void init_public_params() {}
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

// Multilinear fold of host values or points, low variable first, odd tails padded with zero
// (include/ec_operation.cuh:37-55).  Works for Fr and bn128.
template <typename T>
T host_partial_me(T* points, uint inputsize, typename std::vector<Fr>::const_iterator begin,
                  typename std::vector<Fr>::const_iterator end) {
  if (begin >= end) return points[0];
  const uint outputsize = (inputsize + 1) / 2;
  T* new_points = new T[outputsize];
#pragma omp parallel for
  for (int i = 0; i < (int)outputsize; i++) {
    const uint id0 = i * 2, id1 = i * 2 + 1;
    if (id1 < inputsize) new_points[i] = points[id0] + *begin * (points[id1] - points[id0]);
    else new_points[i] = points[id0] - *begin * points[id0];
  }
  T result = host_partial_me(new_points, outputsize, begin + 1, end);
  delete[] new_points;
  return result;
}

// ---- files, timers (include/ioutils.cuh:52-63, include/timer.cuh) ---------------------------------
inline ulong findsize(const std::string& filename) {  // src/ioutils.cu:40-63
  FILE* f = fopen(filename.c_str(), "rb");
  if (!f) {
    fprintf(stderr, "Error: cannot open file %s\n", filename.c_str());
    return 0;
  }
  fseeko(f, 0, SEEK_END);
  const off_t n = ftello(f);
  fclose(f);
  return n < 0 ? 0 : (ulong)n;
}
// The bytes of a device (default) or host buffer, nothing else (src/ioutils.cu:3-38).
inline void savebin(const std::string& filename, const void* data, size_t size, bool is_gpu_data = true) {
  if (!data || size == 0) {
    fprintf(stderr, "Error: Invalid input parameters\n");
    return;
  }
  std::vector<unsigned char> host;
  const void* src = data;
  if (is_gpu_data) {
    host.resize(size);
    grape_veneer::check(grape_d2h(grape_veneer::ctx(), host.data(), data, size));
    src = host.data();
  }
  FILE* f = fopen(filename.c_str(), "wb");
  if (!f) {
    fprintf(stderr, "Error: Failed to open file %s\n", filename.c_str());
    return;
  }
  fwrite(src, 1, size, f);
  fclose(f);
}
// Exactly `size` bytes of a file into a device (default) or host buffer; a short file loads nothing
// (src/ioutils.cu:65-103).
inline void loadbin(const std::string& filename, void* data, size_t size, bool is_gpu_data = true) {
  if (!data || size == 0) {
    fprintf(stderr, "Error: Invalid input parameters\n");
    return;
  }
  FILE* f = fopen(filename.c_str(), "rb");
  if (!f) {
    perror(("Error opening file " + filename).c_str());
    return;
  }
  std::vector<unsigned char> host(size);
  const size_t got = fread(host.data(), 1, size, f);
  fclose(f);
  if (got != size) {
    fprintf(stderr, "Error: Read %zu bytes, expected %lu\n", got, (unsigned long)size);
    return;
  }
  if (is_gpu_data) {
    grape_veneer::check(grape_h2d(grape_veneer::ctx(), data, host.data(), size));
    grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
  } else {
    std::memcpy(data, host.data(), size);
  }
}
// A whole file of int32 values into a fresh device buffer (an old one at *gpu_ptr is freed first);
// returns the element count (src/ioutils.cu:105-124).
inline uint load_data(const std::string& filename, int** gpu_ptr) {
  const ulong n = findsize(filename) / sizeof(int);
  grape_ctx* c = grape_veneer::ctx();
  if (*gpu_ptr) {
    grape_dev_free(c, *gpu_ptr);
    *gpu_ptr = nullptr;
  }
  FILE* f = fopen(filename.c_str(), "rb");
  if (!f) {
    perror(("Error opening file " + filename).c_str());
    exit(1);
  }
  std::vector<int> host(n);
  if (fread(host.data(), sizeof(int), n, f) != n) fprintf(stderr, "Error: short read of %s\n", filename.c_str());
  fclose(f);
  *gpu_ptr = (int*)grape_veneer::dev_alloc(n * sizeof(int));
  grape_veneer::check(grape_h2d(c, *gpu_ptr, host.data(), n * sizeof(int)));
  grape_veneer::check(grape_ctx_sync(c));
  return (uint)n;
}
inline uint load_data(const std::string& filename, int** gpu_ptr, int** cpu_ptr) {  // src/ioutils.cu:126-145
  const ulong n = findsize(filename) / sizeof(int);
  *cpu_ptr = (int*)malloc(sizeof(int) * n);
  FILE* f = fopen(filename.c_str(), "rb");
  if (!f) {
    perror(("Error opening file " + filename).c_str());
    exit(1);
  }
  if (fread(*cpu_ptr, sizeof(int), n, f) != n) fprintf(stderr, "Error: short read of %s\n", filename.c_str());
  fclose(f);
  *gpu_ptr = (int*)grape_veneer::dev_alloc(n * sizeof(int));
  grape_veneer::check(grape_h2d(grape_veneer::ctx(), *gpu_ptr, *cpu_ptr, n * sizeof(int)));
  grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
  return (uint)n;
}
// The one seeded input of the reference: mt19937(123456), uniform over all of int32, into a fresh
// device buffer (src/ioutils.cu:147-170).
inline void generate_data(int** out_ptr, uint size) {
  std::vector<int> h(size);
  std::mt19937 rng(123456);
  std::uniform_int_distribution<int> dist(std::numeric_limits<int>::min(), std::numeric_limits<int>::max());
  for (uint i = 0; i < size; i++) h[i] = dist(rng);
  *out_ptr = (int*)grape_veneer::dev_alloc((size_t)size * sizeof(int));
  grape_veneer::check(grape_h2d(grape_veneer::ctx(), *out_ptr, h.data(), (size_t)size * sizeof(int)));
  grape_veneer::check(grape_ctx_sync(grape_veneer::ctx()));
}

class Timer {  // include/timer.cuh, src/timer.cu: stop() prints milliseconds and returns seconds
 public:
  void start() { start_time = std::chrono::high_resolution_clock::now(); }
  double stop(const std::string& label = "Code block executed") {
    const double s = elapsed();
    printf("\033[35m[Timing]\033[0m %s in: %.3f ms\n", label.c_str(), s * 1000);
    return s;
  }
  double elapsed() {
    auto now = std::chrono::high_resolution_clock::now();
    return std::chrono::duration_cast<std::chrono::microseconds>(now - start_time).count() / 1e6;
  }

 private:
  std::chrono::high_resolution_clock::time_point start_time;
};

#ifndef CPU_TIMER_START
#define CPU_TIMER_START(timer_name) auto timer_name##_start = std::chrono::high_resolution_clock::now();
#define CPU_TIMER_STOP(timer_name)                                                                          \
  do {                                                                                                      \
    auto timer_name##_end = std::chrono::high_resolution_clock::now();                                      \
    double timer_name##_elapsed_ms =                                                                        \
        std::chrono::duration<double, std::milli>(timer_name##_end - timer_name##_start).count();           \
    printf("%s elapsed: %f ms\n", #timer_name, timer_name##_elapsed_ms);                                    \
  } while (0)
#endif
// CUDA_DEBUG of the reference prints the line and the last CUDA error after a device synchronisation;
// here the library's own status plays that part.
#ifndef CUDA_DEBUG
#define CUDA_DEBUG                                                                     \
  do {                                                                                 \
    int grape_rc_ = grape_ctx_sync(grape_veneer::ctx());                               \
    std::cout << __LINE__ << " " << (grape_rc_ == GRAPE_OK ? "no error" : grape_ctx_error(grape_veneer::ctx())) << std::endl; \
  } while (0);
#endif

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
  // a view of `size_` elements somebody else owns (the table tensors of a lookup object)
  static FrTensor view(fr_t* data, uint size_) {
    FrTensor t;
    t.gpu_data = data;
    t.size = t.cap_ = size_;
    t.owned_ = false;
    return t;
  }
  FrTensor(FrTensor&& o) noexcept : gpu_data(o.gpu_data), size(o.size), cap_(o.cap_), owned_(o.owned_) { o.gpu_data = nullptr; }
  ~FrTensor() {
    if (gpu_data && owned_) grape_dev_free(grape_veneer::ctx(), gpu_data);
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
  bool owned_ = true;
  FrTensor() : gpu_data(nullptr), size(0), cap_(0) {}
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
  // The reference declares verify and leaves it empty (src/Hyrax.cu:307-310); its one external check is
  // the pair of identities of test/HyraxTest.cu:88-125, which is what this runs:
  //   c * fold(commitment; row and layer challenges) + commit_d == sum_i z_i G_i
  //   (c * result) * G + commit_ad == z~(low challenges) * G
  // cpu_points: the generators (cpu_points.bin); eval_point: the point the proof was opened at.
  // Throws std::runtime_error when an identity fails.
  void verify(Hyrax_proof& proof, jacob_t* commitment, Fr c, uint size, uint N, const std::vector<Fr>& eval_point,
              const std::vector<bn128>& cpu_points) {
    const uint rows = size / N / com_scale;
    std::vector<bn128> host_commitment(rows);
    grape_veneer::check(grape_d2h(grape_veneer::ctx(), host_commitment.data(), commitment, (size_t)rows * 96));
    const uint start_x = Log2(N * com_scale);
    std::vector<bn128> layer_c(layer_num);
    for (uint i = 0; i < layer_num; i++)
      layer_c[i] = host_partial_me<bn128>(host_commitment.data() + i * (rows / layer_num), rows / layer_num,
                                          eval_point.begin() + start_x, eval_point.end() - Log2(layer_num));
    bn128 C_ = host_partial_me<bn128>(layer_c.data(), layer_num, eval_point.begin() + Log2(size / layer_num), eval_point.end());
    // sum_i z_i G_i on the GPU (one row commitment of z over the same table)
    const uint new_N = (1u << Log2(N)) * com_scale;
    fr_t* d_z = (fr_t*)grape_veneer::dev_alloc((size_t)new_N * 32);
    jacob_t* d_cz = (jacob_t*)grape_veneer::dev_alloc(96);
    grape_veneer::check(grape_h2d(grape_veneer::ctx(), d_z, proof.z, (size_t)new_N * 32));
    grape_veneer::check(grape_commit_fr(grape_veneer::ctx(), table, d_z, new_N, new_N, d_cz));
    bn128 commit_z;
    grape_veneer::check(grape_d2h(grape_veneer::ctx(), commit_z.v, d_cz, 96));
    grape_dev_free(grape_veneer::ctx(), d_z);
    grape_dev_free(grape_veneer::ctx(), d_cz);
    if (!(c * C_ + proof.commit_d == commit_z)) throw std::runtime_error("Hyrax::verify: c * C + com_d != commit(z)");
    const Fr az = host_partial_me<Fr>(proof.z, new_N, eval_point.begin(), eval_point.begin() + start_x);
    if (!((c * proof.result) * cpu_points[0] + proof.commit_ad == az * cpu_points[0]))
      throw std::runtime_error("Hyrax::verify: (c * result) * G + com_ad != z~ * G");
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
// The reference's signature (include/Hyrax.cuh:54): g is its 256-row table over npoints generators.
inline void single_commit(fr_t* d, affine_t* g, jacob_t* com, uint N, uint npoints) {
  grape_table* t = nullptr;
  grape_veneer::check(grape_table_from_reference(grape_veneer::ctx(), g, npoints, &t));
  single_commit(d, t, com, N);
  grape_table_destroy(t);
}

// N random generators [rho_i] * (1, 2) and their table in the reference's layout: `out` receives W = 256
// rows of N affine points, row w = w * G_i, row 0 = infinity (src/ec_operation.cu:15-49, test/ppgen.cu).
// Returns the generators as host points (what the reference saves as cpu_points.bin).
inline std::vector<bn128> precompute_generators(uint N, uint W, affine_t* out) {
  if (W != 256) throw std::runtime_error("precompute_generators: the table has 256 rows");
  grape_ctx* c = grape_veneer::ctx();
  // [rho_i] * (1, 2) as one-scalar commitments over the single base point
  const bn128 base = bn128::one();
  jacob_t* d_base = (jacob_t*)grape_veneer::dev_alloc(96);
  grape_veneer::check(grape_h2d(c, d_base, base.v, 96));
  grape_table* bt = nullptr;
  grape_veneer::check(grape_table_create(c, d_base, 1, 8, 32, &bt));
  std::vector<Fr> rho = random_vec(N);
  fr_t* d_rho = (fr_t*)grape_veneer::dev_alloc((size_t)N * 32);
  jacob_t* d_gens = (jacob_t*)grape_veneer::dev_alloc((size_t)N * 96);
  grape_veneer::check(grape_h2d(c, d_rho, rho.data(), (size_t)N * 32));
  grape_veneer::check(grape_commit_fr(c, bt, d_rho, N, 1, d_gens));
  std::vector<bn128> generators(N);
  grape_veneer::check(grape_d2h(c, generators.data(), d_gens, (size_t)N * 96));
  // magnitudes 1..256 of a 9-bit signed-digit table are the rows 1..256 of the reference layout
  grape_table* t9 = nullptr;
  grape_veneer::check(grape_table_create(c, d_gens, N, 9, 1, &t9));
  grape_veneer::check(grape_dev_zero(c, out, (size_t)N * 64));
  grape_veneer::check(grape_d2d(c, out + N, grape_table_data(t9), (size_t)255 * N * 64));
  grape_veneer::check(grape_ctx_sync(c));
  grape_table_destroy(t9);
  grape_table_destroy(bt);
  grape_dev_free(c, d_rho);
  grape_dev_free(c, d_gens);
  grape_dev_free(c, d_base);
  return generators;
}

// ---- Polynomial (include/polynomial.cuh:8-44, src/polynomial.cu) -----------------------------------
class Polynomial {
 public:
  Polynomial() : c_(1, Fr::zero()) {}
  explicit Polynomial(int degree) : c_(degree + 1, Fr::zero()) {}
  Polynomial(int degree, Fr* coefficients) : c_(coefficients, coefficients + degree + 1) {}
  Polynomial(const Fr& constant) : c_(1, constant) {}
  Polynomial(const std::vector<Fr>& coefficients) : c_(coefficients) {
    if (c_.empty()) c_.push_back(Fr::zero());
  }
  Polynomial operator+(const Polynomial& o) const {
    Polynomial r((int)std::max(c_.size(), o.c_.size()) - 1);
    for (size_t i = 0; i < r.c_.size(); i++) r.c_[i] = at(i) + o.at(i);
    return r;
  }
  Polynomial operator-(const Polynomial& o) const {
    Polynomial r((int)std::max(c_.size(), o.c_.size()) - 1);
    for (size_t i = 0; i < r.c_.size(); i++) r.c_[i] = at(i) - o.at(i);
    return r;
  }
  Polynomial operator*(const Polynomial& o) const {
    Polynomial r((int)(c_.size() + o.c_.size()) - 2);
    for (size_t i = 0; i < c_.size(); i++)
      for (size_t j = 0; j < o.c_.size(); j++) r.c_[i + j] += c_[i] * o.c_[j];
    return r;
  }
  Polynomial operator*(const Fr& val) const {
    Polynomial r(*this);
    for (auto& x : r.c_) x *= val;
    return r;
  }
  Polynomial operator-() const {
    Polynomial r(*this);
    for (auto& x : r.c_) x = -x;
    return r;
  }
  Polynomial& operator+=(const Polynomial& o) { return *this = *this + o; }
  Polynomial& operator-=(const Polynomial& o) { return *this = *this - o; }
  Polynomial& operator*=(const Polynomial& o) { return *this = *this * o; }
  Fr operator()(const Fr& x) const {  // Horner
    Fr acc = Fr::zero();
    for (size_t i = c_.size(); i-- > 0;) acc = acc * x + c_[i];
    return acc;
  }
  Fr operator()(const int& x) const { return (*this)(Fr((long)x)); }
  int getDegree() const { return (int)c_.size() - 1; }
  void setCoefficients(int degree, Fr* coefficients) { c_.assign(coefficients, coefficients + degree + 1); }
  // eq(u, X) = (1 - u) + (2u - 1) X   and   eq(u, v) = uv + (1-u)(1-v)   (src/polynomial.cu:47-53,120-128)
  static Polynomial eq(const Fr& u) { return Polynomial(std::vector<Fr>{Fr::one() - u, u + u - Fr::one()}); }
  static Fr eq(const Fr& u, const Fr& v) { return u * v + (Fr::one() - u) * (Fr::one() - v); }
  friend std::ostream& operator<<(std::ostream& os, const Polynomial& p) {
    os << "Polynomial(degree " << p.getDegree() << ")";
    return os;
  }

 private:
  std::vector<Fr> c_;
  Fr at(size_t i) const { return i < c_.size() ? c_[i] : Fr::zero(); }
};

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
    Fr out;
    grape_veneer::check(grape_lookup_prove_range(grape_veneer::ctx(), handle, S.gpu_data, S.size, A.gpu_data, v.data(),
                                                 (uint32_t)v.size(), 11008, 16384, hyrax.table, msm_size, nullptr, nullptr,
                                                 out.w, nullptr, 0, nullptr));
    double s = 0;
    grape_lookup_last_commit_seconds(handle, &s);
    commit_time += s;   // the reference adds the time of its two commit calls (src/tlookup.cu:319-323)
    return out;
  }
  // The table tensors of include/tlookup.cuh:41-47 as views of the object's device memory: T, B = 1/(T+beta),
  // m (the multiplicities of the last prove).
  FrTensor T() const { return FrTensor::view((fr_t*)grape_lookup_table(handle, 0), table_size()); }
  FrTensor B() const { return FrTensor::view((fr_t*)grape_lookup_table(handle, 1), table_size()); }
  FrTensor m() const { return FrTensor::view((fr_t*)grape_lookup_table(handle, 2), table_size()); }
  uint table_size() const {
    uint32_t n = 0;
    grape_lookup_params(handle, nullptr, nullptr, nullptr, &n);
    return n;
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
  // the reference's constructor: the int32 table f comes from a file of len values (src/tlookup.cu:350-371)
  tLookupRangeMapping(const int low_, const uint len, const std::string& filename) : low(low_), handle(nullptr) {
    int* d_map = (int*)grape_veneer::dev_alloc((size_t)len * sizeof(int));
    loadbin(filename, d_map, (size_t)len * sizeof(int));
    grape_veneer::check(grape_lookup_mapping_create(grape_veneer::ctx(), low_, len, d_map, &handle));
    grape_lookup_params(handle, alpha.w, beta.w, r.w, nullptr);
    grape_dev_free(grape_veneer::ctx(), d_map);
  }
  ~tLookupRangeMapping() { grape_lookup_destroy(handle); }
  tLookupRangeMapping(const tLookupRangeMapping&) = delete;
  Fr prove(FrTensor& S_in, FrTensor& S_out, FrTensor& A, const std::vector<Fr>& v, Hyrax& hyrax, uint msm_size,
           double& commit_time) {
    FrTensor work(1u << Log2(S_in.size));
    Fr out;
    grape_veneer::check(grape_lookup_prove_mapping(grape_veneer::ctx(), handle, S_in.gpu_data, S_out.gpu_data, S_in.size,
                                                   work.gpu_data, A.gpu_data, v.data(), (uint32_t)v.size(), 11008, 16384,
                                                   hyrax.table, msm_size, nullptr, nullptr, out.w, nullptr, 0, nullptr));
    double s = 0;
    grape_lookup_last_commit_seconds(handle, &s);
    commit_time += s;
    return out;
  }
};
