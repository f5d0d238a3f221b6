// Internal definitions behind the opaque handles of the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/grape_b200.h"
#include "rng.cuh"

struct grape_table;

struct grape_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  // second stream + events: host-to-device copies of the host-buffer entry points overlap compute
  cudaStream_t copy_stream = nullptr;
  std::vector<cudaEvent_t> copy_events;
  // events of grape_h2d_prefetch, indexed by ticket; free_tickets lists the ones that were waited for
  std::vector<cudaEvent_t> prefetch_events;
  std::vector<uint32_t> free_tickets;
  // scratch arena: a bump allocator over a few device blocks.  A top-level call resets it,
  // carves what its kernels need, and the next call on the stream reuses the same memory.
  struct ArenaBlock { void* ptr; size_t size; size_t off; };
  std::vector<ArenaBlock> arena;
  // pinned staging buffer for the host-buffer entry points
  void* pinned = nullptr;
  size_t pinned_bytes = 0;
  void* dstage = nullptr;
  size_t dstage_bytes = 0;
  grape::RngState rng;   // prover randomness: OS-keyed ChaCha20, or the seeded test stream
  // device status word: kernels OR a GRAPE_STATUS_* bit into it instead of trapping
  uint32_t* d_status = nullptr;
  std::string err;
  int sm_count = 148;
  // commitments of a lookup's A by the bucket method: 0 never, 1 when the cost model favours it, 2 whenever supported
  int bucket_mode = 1;
  // accumulation of commitments with affine accumulators: 0 never, 1 when the cost model favours it,
  // 2 always with affine_b slots per lane and affine_chunks chunks per row block (0 = chosen).  Kept
  // apart for int32 scalars (default 0) and Fr scalars (default 1: the lookups' A tensors, where the
  // planner's choice was measured to take 8 % off a layer proof).
  int affine_mode = 0;
  int affine_mode_fr = 1;
  int affine_b = 0, affine_chunks = 0;
  // fixed-base table of the opening protocol's point G (one generator, 16 x 16-bit windows), built on
  // the first opening and rebuilt when another G is passed; g_key: the 96 bytes of that G
  grape_table* g_table = nullptr;
  unsigned char g_key[96] = {0};
  // launch counters (own kernels launched since creation), read by the benchmark
  uint64_t launches = 0;
  // wall-clock bracket on the stream (grape_timer_begin / grape_timer_end)
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  // optional per-kernel timing of the dominant kernel of a call (commit_accumulate, ...):
  // event pairs recorded around it while `profile` is set, summed by grape_prof_read
  bool profile = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events;
};

struct grape_table {
  grape_ctx* ctx = nullptr;
  void* data = nullptr;  // affine records
  bool owned = false;
  uint32_t n_gens = 0;
  uint32_t window_bits = 8;
  uint32_t n_windows = 1;
  uint32_t n_digits = 128;      // addressable magnitudes per window: 1..n_digits
  uint64_t window_stride = 0;   // records between consecutive windows
  uint32_t first_digit_row = 0; // row holding magnitude 1 (1 for the reference's 256-row layout)
  uint32_t curve = 0;           // GRAPE_CURVE_BN254 or GRAPE_CURVE_BLS12_381
};

namespace grape {

// Brackets the dominant kernel of a call with events when profiling is on.
struct ProfScope {
  grape_ctx* ctx;
  cudaEvent_t a = nullptr, b = nullptr;
  explicit ProfScope(grape_ctx* c) : ctx(c) {
    if (ctx->profile) {
      cudaEventCreate(&a);
      cudaEventCreate(&b);
      cudaEventRecord(a, ctx->stream);
    }
  }
  ~ProfScope() {
    if (a) {
      cudaEventRecord(b, ctx->stream);
      ctx->prof_events.push_back({a, b});
    }
  }
};

constexpr uint32_t STATUS_DIGIT_RANGE = 1u;  // a scalar exceeded the declared max_bits
constexpr uint32_t STATUS_HIST_RANGE = 2u;   // a lookup query fell outside the table
constexpr uint32_t STATUS_PIPE_TIMEOUT = 4u; // a bounded wait on a shared-memory copy pipeline ran out

// Every entry point that takes a context makes the context's GPU the calling thread's current
// device first (allocations and launches would otherwise land on whatever device the caller, or
// another library in the process, selected last) and leaves it current.
inline void make_device_current(const grape_ctx* ctx) {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d != ctx->device) cudaSetDevice(ctx->device);
}

inline int fail(grape_ctx* ctx, int code, const std::string& msg) {
  if (ctx) ctx->err = msg;
  return code;
}

#define GRAPE_CUDA_TRY(ctx, expr)                                                         \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      return grape::fail((ctx), GRAPE_ERR_CUDA,                                           \
                         std::string(#expr) + ": " + cudaGetErrorString(_e));             \
    }                                                                                     \
  } while (0)

// Starts a new top-level call: everything handed out before is up for reuse (stream order keeps
// earlier kernels safe).  Several blocks left by a call that outgrew the arena are merged into one.
inline int arena_reset(grape_ctx* ctx) {
  if (ctx->arena.size() > 1) {
    GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    size_t total = 0;
    for (auto& b : ctx->arena) { total += b.size; cudaFree(b.ptr); }
    ctx->arena.clear();
    void* p = nullptr;
    if (cudaMalloc(&p, total) == cudaSuccess) ctx->arena.push_back({p, total, 0});
    else cudaGetLastError();
  }
  for (auto& b : ctx->arena) b.off = 0;
  return GRAPE_OK;
}

// Hands out `bytes` of scratch (256-byte aligned), adding a device block when the arena is full.
inline int arena_alloc(grape_ctx* ctx, size_t bytes, void** out) {
  bytes = (bytes + 255) & ~size_t(255);
  if (bytes == 0) bytes = 256;
  for (auto& b : ctx->arena) {
    if (b.off + bytes <= b.size) {
      *out = reinterpret_cast<char*>(b.ptr) + b.off;
      b.off += bytes;
      return GRAPE_OK;
    }
  }
  size_t want = bytes < (size_t(32) << 20) ? (size_t(32) << 20) : bytes;
  void* p = nullptr;
  if (cudaMalloc(&p, want) != cudaSuccess) {
    cudaGetLastError();
    return fail(ctx, GRAPE_ERR_NOMEM, "scratch arena allocation failed");
  }
  ctx->arena.push_back({p, want, bytes});
  *out = p;
  return GRAPE_OK;
}

template <class T>
inline int arena_alloc_t(grape_ctx* ctx, size_t count, T** out) {
  void* p = nullptr;
  int rc = arena_alloc(ctx, count * sizeof(T), &p);
  *out = reinterpret_cast<T*>(p);
  return rc;
}

inline uint32_t log2ceil(uint64_t n) {  // the reference's Log2 (src/ioutils.cu:173-190)
  if (n == 0) return 0;
  n--;
  uint32_t r = 0;
  while (n > 0) { n >>= 1; r++; }
  return r;
}

}  // namespace grape
