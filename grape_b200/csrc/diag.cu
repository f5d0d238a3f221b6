// Measured integer-pipe ceilings used as roofline denominators for the multiplication-bound
// kernels: dependent-free multiply-add loops at full occupancy, timed with CUDA events.
//   kind 0: mad.lo.u32           (32-bit multiply-add, one result word)
//   kind 1: mad.wide.u32         (32x32 -> 64-bit multiply-add)
//   kind 2: mad.lo.cc + madc.hi  (the lo/hi pair form the field arithmetic is written in)
//   kind 3: Montgomery multiplications in Fp (field muls per second)
//   kind 4: the same with a 16-product loop body;  kind 5: dedicated squarings in Fp
#include "ctx.cuh"
#include "curve.cuh"

namespace grape {

// Mixed additions on register-resident data (no table, no scalars): the arithmetic ceiling of the
// commitment inner loop at its own register budget.
__global__ void __launch_bounds__(128, 4) k_madd_peak(const uint32_t* __restrict__ seed_pts, uint32_t* sink, int iters) {
  Affine q = Affine::load(seed_pts + (threadIdx.x & 7) * 16);
  Xyzz acc = Xyzz::from_affine(Affine::load(seed_pts + 8 * 16 + (threadIdx.x & 7) * 16));
  for (int it = 0; it < iters; it++) {
    xyzz_madd_lazy(acc, q);              // the addition the commitment kernel runs (lazy residues)
    q.x = fe_canon(acc.zz);              // keep the operands changing; values need not be curve points for timing
  }
  if (acc.x.v[0] == 0x12345 && acc.y.v[1] == 7) sink[0] = acc.zz.v[2];
}

constexpr int PEAK_ITERS = 2048;
constexpr int PEAK_CHAINS = 8;

template <int KIND>
__global__ void __launch_bounds__(256) k_int_peak(uint32_t* sink, uint32_t seed) {
  uint32_t a = seed + threadIdx.x, b = seed * 3 + blockIdx.x;
  if (KIND == 0) {
    uint32_t acc[PEAK_CHAINS];
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) acc[k] = a + k;
    for (int it = 0; it < PEAK_ITERS; it++) {
#pragma unroll
      for (int k = 0; k < PEAK_CHAINS; k++)
        asm volatile("mad.lo.u32 %0, %1, %2, %0;" : "+r"(acc[k]) : "r"(a), "r"(b));
    }
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) s ^= acc[k];
    if (s == 0x12345) sink[0] = s;
  } else if (KIND == 1) {
    unsigned long long acc[PEAK_CHAINS];
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) acc[k] = a + k;
    for (int it = 0; it < PEAK_ITERS; it++) {
#pragma unroll
      for (int k = 0; k < PEAK_CHAINS; k++)
        asm volatile("mad.wide.u32 %0, %1, %2, %0;" : "+l"(acc[k]) : "r"(a), "r"(b));
    }
    unsigned long long s = 0;
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) s ^= acc[k];
    if (s == 0x12345) sink[0] = (uint32_t)s;
  } else if (KIND == 2) {
    uint32_t lo[PEAK_CHAINS], hi[PEAK_CHAINS];
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) { lo[k] = a + k; hi[k] = b + k; }
    for (int it = 0; it < PEAK_ITERS; it++) {
#pragma unroll
      for (int k = 0; k < PEAK_CHAINS; k++)
        asm volatile("mad.lo.cc.u32 %0, %2, %3, %0;\n\tmadc.hi.u32 %1, %2, %3, %1;"
                     : "+r"(lo[k]), "+r"(hi[k]) : "r"(a), "r"(b));
    }
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < PEAK_CHAINS; k++) s ^= lo[k] ^ hi[k];
    if (s == 0x12345) sink[0] = s;
  } else if (KIND == 4) {
    // the same multiplications with a loop body of 16 inlined products (about 3 000 instructions),
    // the footprint of one mixed point addition: exposes instruction-fetch limits
    Fp x[4], y;
#pragma unroll
    for (int i = 0; i < 8; i++) { x[0].v[i] = a + i; x[1].v[i] = b + i; x[2].v[i] = a * 3 + i; x[3].v[i] = b * 5 + i; y.v[i] = (a ^ b) + i; }
#pragma unroll
    for (int k = 0; k < 4; k++) x[k].v[7] &= 0x0fffffffu;
    y.v[7] &= 0x0fffffffu;
    for (int it = 0; it < PEAK_ITERS / 64; it++) {
#pragma unroll
      for (int r = 0; r < 4; r++) {
        x[0] = fe_mul(x[0], y);
        x[1] = fe_mul(x[1], x[0]);
        x[2] = fe_mul(x[2], y);
        x[3] = fe_mul(x[3], x[2]);
      }
    }
    if (x[0].v[0] == 0x12345 && x[1].v[3] == 7 && x[3].v[2] == 9) sink[0] = x[0].v[1];
  } else if (KIND == 5) {
    // dedicated squarings, two independent chains per thread
    Fp x[2];
#pragma unroll
    for (int i = 0; i < 8; i++) { x[0].v[i] = a + i; x[1].v[i] = b + i; }
    x[0].v[7] &= 0x0fffffffu; x[1].v[7] &= 0x0fffffffu;
    for (int it = 0; it < PEAK_ITERS / 8; it++) {
      x[0] = fe_sqr(x[0]);
      x[1] = fe_sqr(x[1]);
    }
    if (x[0].v[0] == 0x12345 && x[1].v[3] == 7) sink[0] = x[0].v[1];
  } else {
    Fp x[2], y;
#pragma unroll
    for (int i = 0; i < 8; i++) { x[0].v[i] = a + i; x[1].v[i] = b + i; y.v[i] = (a ^ b) + i; }
    x[0].v[7] &= 0x0fffffffu; x[1].v[7] &= 0x0fffffffu; y.v[7] &= 0x0fffffffu;
    for (int it = 0; it < PEAK_ITERS / 8; it++) {
      x[0] = fe_mul(x[0], y);
      x[1] = fe_mul(x[1], y);
    }
    if (x[0].v[0] == 0x12345 && x[1].v[3] == 7) sink[0] = x[0].v[1];
  }
}

// Identities that tie the specialised field routines to the plain multiplication, element by element:
//   dedicated squaring == a * a,   division-step inverse == Fermat inverse == Euclid inverse,
//   a * a^-1 == 1   (a != 0).
template <class F>
__global__ void k_field_check(const uint32_t* __restrict__ in, uint64_t n, uint32_t* __restrict__ bad) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const F a = F::load(in + i * F::N);
  uint32_t fails = 0;
  if (fe_sqr(a) != fe_mul(a, a)) fails |= 1u;
  const F inv = fe_inv(a);
  if (inv != fe_inv_fermat(a)) fails |= 2u;
  if (inv != fe_inv_kaliski(a)) fails |= 16u;
  if (!a.is_zero() && fe_mul(a, inv) != F::one()) fails |= 4u;
  if (a.is_zero() && !inv.is_zero()) fails |= 8u;
  if (fails) atomicOr(bad, fails);
}

}  // namespace grape

using namespace grape;

// field: 0 BN254 Fp, 1 BN254 Fr, 2 BLS12-381 Fp, 3 BLS12-381 Fr.  d_elems: n canonical Montgomery elements
// (8 or 12 limbs each).  *h_fail_mask = OR over the elements of: 1 squaring differs from a*a, 2 the
// inverse (batched division steps) differs from the Fermat inverse, 4 a * a^-1 != 1, 8 the inverse of 0
// is not 0, 16 the inverse differs from the binary-Euclid inverse.
extern "C" int grape_diag_field_check(grape_ctx* ctx, int field, const void* d_elems, uint64_t n,
                                      uint32_t* h_fail_mask) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !h_fail_mask || field < 0 || field > 3 || (!d_elems && n)) return GRAPE_ERR_INVALID;
  arena_reset(ctx);
  uint32_t* bad = nullptr;
  int rc = arena_alloc_t(ctx, 64, &bad);
  if (rc) return rc;
  GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(bad, 0, 4, ctx->stream));
  if (n) {
    const uint32_t blocks = (uint32_t)((n + 63) / 64);
    const uint32_t* in = reinterpret_cast<const uint32_t*>(d_elems);
    if (field == 0) k_field_check<Fp><<<blocks, 64, 0, ctx->stream>>>(in, n, bad);
    else if (field == 1) k_field_check<Fr><<<blocks, 64, 0, ctx->stream>>>(in, n, bad);
    else if (field == 2) k_field_check<BlsFp><<<blocks, 64, 0, ctx->stream>>>(in, n, bad);
    else k_field_check<BlsFr><<<blocks, 64, 0, ctx->stream>>>(in, n, bad);
    ctx->launches += 1;
  }
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_fail_mask, bad, 4, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

// Writes operations per second: kinds 0-2 count multiply-add instructions (a lo/hi pair counts 2),
// kind 3 counts field multiplications.
extern "C" int grape_measure_int_peak(grape_ctx* ctx, int kind, double* ops_per_second) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !ops_per_second || kind < 0 || kind > 5) return GRAPE_ERR_INVALID;
  arena_reset(ctx);
  uint32_t* sink = nullptr;
  int rc = arena_alloc_t(ctx, 64, &sink);
  if (rc) return rc;
  const int blocks = ctx->sm_count * 8, threads = 256;
  cudaEvent_t e0, e1;
  GRAPE_CUDA_TRY(ctx, cudaEventCreate(&e0));
  GRAPE_CUDA_TRY(ctx, cudaEventCreate(&e1));
  float best = 1e30f;
  for (int rep = 0; rep < 4; rep++) {
    cudaEventRecord(e0, ctx->stream);
    if (kind == 0) k_int_peak<0><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    else if (kind == 1) k_int_peak<1><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    else if (kind == 2) k_int_peak<2><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    else if (kind == 3) k_int_peak<3><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    else if (kind == 4) k_int_peak<4><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    else k_int_peak<5><<<blocks, threads, 0, ctx->stream>>>(sink, rep + 1);
    cudaEventRecord(e1, ctx->stream);
    ctx->launches += 1;
    GRAPE_CUDA_TRY(ctx, cudaEventSynchronize(e1));
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  double per_thread;
  if (kind == 0 || kind == 1) per_thread = (double)PEAK_ITERS * PEAK_CHAINS;
  else if (kind == 2) per_thread = 2.0 * PEAK_ITERS * PEAK_CHAINS;
  else if (kind == 3 || kind == 5) per_thread = 2.0 * (PEAK_ITERS / 8);
  else per_thread = 16.0 * (PEAK_ITERS / 64);
  *ops_per_second = per_thread * blocks * threads / (best * 1e-3);
  return GRAPE_OK;
}

// Mixed XYZZ additions per second on register-resident operands (kind of ceiling for the
// commitment kernel: same code, same launch bounds, no memory traffic).
extern "C" int grape_measure_madd_peak(grape_ctx* ctx, double* adds_per_second) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !adds_per_second) return GRAPE_ERR_INVALID;
  arena_reset(ctx);
  uint32_t* buf = nullptr;
  int rc = arena_alloc_t(ctx, 16 * 16 + 64, &buf);
  if (rc) return rc;
  uint32_t h[16 * 16];
  for (int i = 0; i < 16 * 16; i++) h[i] = (0x9E3779B9u * (i + 1)) & ((i % 8 == 7) ? 0x0fffffffu : 0xffffffffu);
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(buf, h, sizeof h, cudaMemcpyHostToDevice, ctx->stream));
  const int blocks = ctx->sm_count * 4, threads = 128, iters = 512;
  cudaEvent_t e0, e1;
  GRAPE_CUDA_TRY(ctx, cudaEventCreate(&e0));
  GRAPE_CUDA_TRY(ctx, cudaEventCreate(&e1));
  float best = 1e30f;
  for (int rep = 0; rep < 4; rep++) {
    cudaEventRecord(e0, ctx->stream);
    k_madd_peak<<<blocks, threads, 0, ctx->stream>>>(buf, buf + 16 * 16, iters);
    cudaEventRecord(e1, ctx->stream);
    ctx->launches += 1;
    GRAPE_CUDA_TRY(ctx, cudaEventSynchronize(e1));
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  *adds_per_second = (double)iters * blocks * threads / (best * 1e-3);
  return GRAPE_OK;
}
