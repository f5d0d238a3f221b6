// Context, memory and RNG entry points of the C ABI.
#include <cstring>
#include <vector>

#include <sys/random.h>
#include <cstdio>

#include "ctx.cuh"
#include "hostfr.hpp"

using namespace grape;

extern "C" int grape_version(void) { return 2; }

namespace grape {
bool rng_os_key(RngKey* key) {
  unsigned char* p = reinterpret_cast<unsigned char*>(key->k);
  size_t got = 0;
  while (got < sizeof key->k) {
    ssize_t r = getrandom(p + got, sizeof key->k - got, 0);
    if (r <= 0) break;
    got += (size_t)r;
  }
  if (got == sizeof key->k) return true;
  FILE* f = fopen("/dev/urandom", "rb");
  if (!f) return false;
  const size_t n = fread(p, 1, sizeof key->k, f);
  fclose(f);
  return n == sizeof key->k;
}
}  // namespace grape

extern "C" int grape_ctx_create(int device, grape_ctx** out) {
  if (!out) return GRAPE_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n)
    return GRAPE_ERR_CUDA;  // no usable GPU: there is deliberately no CPU fallback
  grape_ctx* ctx = new grape_ctx();
  ctx->device = device;
  if (cudaSetDevice(device) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete ctx;
    return GRAPE_ERR_CUDA;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
  if (cudaMalloc(&ctx->d_status, 64) != cudaSuccess) {
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return GRAPE_ERR_NOMEM;
  }
  cudaMemsetAsync(ctx->d_status, 0, 64, ctx->stream);
  // blinders and challenges come from ChaCha20 under an OS-drawn key unless grape_rng_seed is called
  if (!rng_os_key(&ctx->rng.key)) {
    cudaFree(ctx->d_status);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return GRAPE_ERR_INVALID;  // no entropy source: refuse rather than fall back to a fixed stream
  }
  *out = ctx;
  return GRAPE_OK;
}

extern "C" int grape_ctx_destroy(grape_ctx* ctx) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->g_table) grape_table_destroy(ctx->g_table);
  for (auto& b : ctx->arena) cudaFree(b.ptr);
  if (ctx->dstage) cudaFree(ctx->dstage);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  for (auto e : ctx->copy_events) cudaEventDestroy(e);
  for (auto e : ctx->prefetch_events) cudaEventDestroy(e);
  if (ctx->t0) { cudaEventDestroy(ctx->t0); cudaEventDestroy(ctx->t1); }
  for (auto& pr : ctx->prof_events) { cudaEventDestroy(pr.first); cudaEventDestroy(pr.second); }
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return GRAPE_OK;
}

extern "C" const char* grape_ctx_error(const grape_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

extern "C" int grape_ctx_sync(grape_ctx* ctx) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return GRAPE_OK;
}

extern "C" void* grape_ctx_stream(grape_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

extern "C" uint64_t grape_ctx_launches(const grape_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int grape_ctx_status(grape_ctx* ctx, uint32_t* flags) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !flags) return GRAPE_ERR_INVALID;
  uint32_t h = 0;
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&h, ctx->d_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  if (h) GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_status, 0, 4, ctx->stream));
  *flags = h;
  return GRAPE_OK;
}

extern "C" int grape_rng_seed(grape_ctx* ctx, uint64_t seed) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  ctx->rng.seeded = true;   // the replayable 64-bit test stream (see rng.cuh): not for production proofs
  ctx->rng.splitmix = splitmix_init(seed, 0);
  return GRAPE_OK;
}

extern "C" int grape_rng_fr(grape_ctx* ctx, void* h_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || (!h_out && n)) return GRAPE_ERR_INVALID;
  HostFr* o = reinterpret_cast<HostFr*>(h_out);
  for (uint64_t i = 0; i < n; i++) o[i] = rng_draw_fr(ctx->rng);
  return GRAPE_OK;
}

extern "C" int grape_dev_alloc(grape_ctx* ctx, size_t bytes, void** d_out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_out) return GRAPE_ERR_INVALID;
  *d_out = nullptr;
  if (bytes == 0) return GRAPE_OK;
  cudaError_t e = cudaMalloc(d_out, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ctx, GRAPE_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  }
  return GRAPE_OK;
}

extern "C" int grape_dev_free(grape_ctx* ctx, void* d_ptr) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (!d_ptr) return GRAPE_OK;
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaFree(d_ptr));
  return GRAPE_OK;
}

extern "C" int grape_h2d(grape_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (bytes == 0) return GRAPE_OK;
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  // pageable sources are staged by the runtime before the call returns; pinned ones are not,
  // so callers that reuse a pinned source must grape_ctx_sync() first.
  return GRAPE_OK;
}

// Host-to-device copy on the context's copy stream, so that it overlaps the kernels of the main
// stream; h_src should be page-locked (a pageable source makes the call synchronous).  The copy
// starts once the work already queued on the main stream is done (the destination may still be in
// use by it).  *ticket identifies the copy for grape_prefetch_wait, which makes the main stream wait
// for that copy (and releases the ticket).
extern "C" int grape_h2d_prefetch(grape_ctx* ctx, void* d_dst, const void* h_src, size_t bytes, uint32_t* ticket) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !ticket) return GRAPE_ERR_INVALID;
  if (!ctx->copy_stream) GRAPE_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  if (ctx->copy_events.empty()) {
    cudaEvent_t e;
    GRAPE_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    ctx->copy_events.push_back(e);
  }
  uint32_t tk;
  if (!ctx->free_tickets.empty()) {
    tk = ctx->free_tickets.back();
    ctx->free_tickets.pop_back();
  } else {
    cudaEvent_t e;
    GRAPE_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    ctx->prefetch_events.push_back(e);
    tk = (uint32_t)ctx->prefetch_events.size() - 1;
  }
  GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[0], ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_events[0], 0));
  if (bytes) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->prefetch_events[tk], ctx->copy_stream));
  *ticket = tk;
  return GRAPE_OK;
}

extern "C" int grape_prefetch_wait(grape_ctx* ctx, uint32_t ticket) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || ticket >= ctx->prefetch_events.size()) return GRAPE_ERR_INVALID;
  GRAPE_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->prefetch_events[ticket], 0));
  ctx->free_tickets.push_back(ticket);
  return GRAPE_OK;
}

extern "C" int grape_d2h(grape_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (bytes)
    GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return GRAPE_OK;
}

extern "C" int grape_d2d(grape_ctx* ctx, void* d_dst, const void* d_src, size_t bytes) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (bytes)
    GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return GRAPE_OK;
}

extern "C" int grape_dev_zero(grape_ctx* ctx, void* d_dst, size_t bytes) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (bytes) GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(d_dst, 0, bytes, ctx->stream));
  return GRAPE_OK;
}

extern "C" int grape_host_alloc_pinned(grape_ctx* ctx, size_t bytes, void** h_out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !h_out) return GRAPE_ERR_INVALID;
  cudaError_t e = cudaMallocHost(h_out, bytes);
  if (e != cudaSuccess) return fail(ctx, GRAPE_ERR_NOMEM, "cudaMallocHost failed");
  return GRAPE_OK;
}

extern "C" int grape_host_device_pointer(grape_ctx* ctx, const void* h_ptr, void** d_out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !h_ptr || !d_out) return GRAPE_ERR_INVALID;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, h_ptr) != cudaSuccess || attr.type != cudaMemoryTypeHost || !attr.devicePointer) {
    cudaGetLastError();
    return fail(ctx, GRAPE_ERR_INVALID, "not a page-locked host buffer");
  }
  *d_out = attr.devicePointer;
  return GRAPE_OK;
}

extern "C" int grape_host_free_pinned(grape_ctx* ctx, void* h_ptr) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (h_ptr) GRAPE_CUDA_TRY(ctx, cudaFreeHost(h_ptr));
  return GRAPE_OK;
}

// ---- timing helpers (CUDA events on the context's stream) --------------------------------------
extern "C" int grape_timer_begin(grape_ctx* ctx) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  if (!ctx->t0) {
    GRAPE_CUDA_TRY(ctx, cudaEventCreate(&ctx->t0));
    GRAPE_CUDA_TRY(ctx, cudaEventCreate(&ctx->t1));
  }
  GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->t0, ctx->stream));
  return GRAPE_OK;
}

extern "C" int grape_timer_end(grape_ctx* ctx, float* ms) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !ms || !ctx->t0) return GRAPE_ERR_INVALID;
  GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->t1, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaEventSynchronize(ctx->t1));
  GRAPE_CUDA_TRY(ctx, cudaEventElapsedTime(ms, ctx->t0, ctx->t1));
  return GRAPE_OK;
}

extern "C" int grape_lookup_set_bucket_commit(grape_ctx* ctx, int mode) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || mode < 0 || mode > 2) return GRAPE_ERR_INVALID;
  ctx->bucket_mode = mode;
  return GRAPE_OK;
}

extern "C" int grape_commit_set_affine(grape_ctx* ctx, int mode, int slots_per_lane, int chunks) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || mode < -1 || mode > 2 || slots_per_lane < 0 || slots_per_lane > 64 || chunks < 0)
    return GRAPE_ERR_INVALID;
  ctx->affine_mode = mode < 0 ? 0 : mode;     // -1: back to what a new context starts with
  ctx->affine_mode_fr = mode < 0 ? 1 : mode;
  ctx->affine_b = slots_per_lane;
  ctx->affine_chunks = chunks;
  return GRAPE_OK;
}

extern "C" int grape_prof_enable(grape_ctx* ctx, int on) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  ctx->profile = on != 0;
  return GRAPE_OK;
}

// Sums and clears the recorded dominant-kernel intervals.
extern "C" int grape_prof_read(grape_ctx* ctx, float* total_ms, uint32_t* count) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !total_ms || !count) return GRAPE_ERR_INVALID;
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  float sum = 0;
  for (auto& pr : ctx->prof_events) {
    float ms = 0;
    cudaEventElapsedTime(&ms, pr.first, pr.second);
    sum += ms;
    cudaEventDestroy(pr.first);
    cudaEventDestroy(pr.second);
  }
  *total_ms = sum;
  *count = (uint32_t)ctx->prof_events.size();
  ctx->prof_events.clear();
  return GRAPE_OK;
}

// ---- host-side Fr arithmetic for callers that used libff's Fr --------------------------------
// (the reference does its claim algebra on the host with libff; these keep a drop-in veneer free
// of any arithmetic of its own).  All pointers are host pointers to 32-byte Montgomery elements.
extern "C" void grape_hfr_add(const void* a, const void* b, void* out) {
  *reinterpret_cast<HostFr*>(out) = fr_add(*reinterpret_cast<const HostFr*>(a), *reinterpret_cast<const HostFr*>(b));
}
extern "C" void grape_hfr_sub(const void* a, const void* b, void* out) {
  *reinterpret_cast<HostFr*>(out) = fr_sub(*reinterpret_cast<const HostFr*>(a), *reinterpret_cast<const HostFr*>(b));
}
extern "C" void grape_hfr_mul(const void* a, const void* b, void* out) {
  *reinterpret_cast<HostFr*>(out) = fr_mul(*reinterpret_cast<const HostFr*>(a), *reinterpret_cast<const HostFr*>(b));
}
extern "C" void grape_hfr_inv(const void* a, void* out) {
  *reinterpret_cast<HostFr*>(out) = fr_inv(*reinterpret_cast<const HostFr*>(a));
}
extern "C" void grape_hfr_from_i64(int64_t v, void* out) { *reinterpret_cast<HostFr*>(out) = fr_from_i64(v); }
