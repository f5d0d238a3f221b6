// LogUp-style lookup argument ("tlookup") for range tables and (x, f(x)) mapping tables.
//
// Replaces (paths inside the reference project):
//   get_histogram_kernel, tlookuprange_init_kernel, tLookupRangeMapping_init_kernel,
//   tlookup_inv_kernel, tLookup_poly_kernel, tLookup_poly_sum_kernel,
//   tLookup_phase2_reduce_kernel                               src/tlookup.cu:5-113
//   tLookup_phase1/2 and their step polynomials                src/tlookup.cu:117-244
//   tLookup / tLookupRange / tLookupRangeMapping                src/tlookup.cu:247-456
//
// As in the sumcheck provers, all challenges are inputs (v) or drawn up front from the context's
// random stream (alpha, r, u), so every round is enqueued without waiting for the host: one fused
// kernel per round accumulates the round's sums and folds the tensors in place, the sums of all
// rounds return in one copy, and the host assembles the round polynomials and runs the reference's
// checks.  Inversions are batched (Montgomery's trick) instead of one extended-Euclid per element.
#include <algorithm>
#include <cstring>
#include <vector>

#include "ctx.cuh"
#include "field.cuh"
#include "hostfr.hpp"

struct grape_lookup {
  grape_ctx* ctx = nullptr;
  int32_t low = 0;
  uint32_t n = 0;          // table size (power of two)
  bool mapping = false;
  grape::HostFr alpha, beta, r;
  uint32_t* T = nullptr;   // table values (Fr)
  uint32_t* B = nullptr;   // 1 / (T + beta)
  uint32_t* m = nullptr;   // multiplicities of the last prove (Fr)
  uint32_t* mapped = nullptr;  // f(x) as Fr (mapping tables)
  uint32_t* hist = nullptr;    // u32 bins
  // what a verifier of the last proof needs besides the round polynomials: the prover's u and the
  // five tensors folded down to one value each, A~(v), S~(v), B~(v2), T~(v2), m~(v2)
  std::vector<grape::HostFr> last_u;
  grape::HostFr last_finals[5];
  bool has_last = false;
  // device time of the commitments of A and m inside the last prove (the reference reports it through
  // its commit_time argument, src/tlookup.cu:319-323)
  cudaEvent_t ev_commit0 = nullptr, ev_commit1 = nullptr;
  float last_commit_ms = 0.f;
};

namespace grape {

void eq_weights_async(grape_ctx* ctx, const void* d_x, uint32_t nv, uint32_t c, void* d_w);
int fr_sum_async(grape_ctx* ctx, const void* d_in, uint64_t n, void* d_out);
int fr_inverse_async(grape_ctx* ctx, const void* d_in, const void* d_shift, void* d_out, uint64_t n);
int commit_fr_padded_async(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size, uint32_t wd,
                           uint32_t inner, uint32_t inner_pad, const void* d_const, void* d_out);
int constant_columns_point_async(grape_ctx* ctx, const grape_table* t, uint32_t wd, uint32_t inner, uint32_t inner_pad,
                                 const void* d_const, uint32_t** d_point);
int commit_gathered_async(grape_ctx* ctx, const grape_table* t, const uint32_t* d_idx, const uint32_t* d_B,
                          uint32_t n_bins, uint64_t size, uint32_t wd, const void* d_extra, void* d_out);
int commit_fr_async(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size, uint32_t wd,
                    void* d_out);

constexpr int LT = 128;

template <int NS>
__device__ __forceinline__ void lk_block_reduce_store(Fr (&acc)[NS], uint32_t* __restrict__ dst) {
  __shared__ Fr part[LT / 32][NS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int s = 0; s < NS; s++) {
    Fr v = acc[s];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fe_add(v, fe_shfl_down(v, off));
    if (lane == 0) part[warp][s] = v;
  }
  __syncthreads();
  if (threadIdx.x < NS) {
    Fr v = part[0][threadIdx.x];
    for (int w = 1; w < LT / 32; w++) v = fe_add(v, part[w][threadIdx.x]);
    v.store(dst + threadIdx.x * 8);
  }
}

template <int NS>
__global__ void __launch_bounds__(LT) k_lk_reduce(const uint32_t* __restrict__ partial, uint32_t n_blocks,
                                                  uint32_t* __restrict__ dst) {
  Fr acc[NS];
#pragma unroll
  for (int s = 0; s < NS; s++) acc[s] = Fr::zero();
  for (uint32_t b = threadIdx.x; b < n_blocks; b += LT) {
#pragma unroll
    for (int s = 0; s < NS; s++) acc[s] = fe_add(acc[s], Fr::load_nc(partial + ((uint64_t)b * NS + s) * 8));
  }
  lk_block_reduce_store<NS>(acc, dst);
}

// T[i] = low + i (+ r * map[i]),  B[i] = 1 / (T[i] + beta) is filled by a batched inversion afterwards.
__global__ void k_table_init(uint32_t* __restrict__ T, const uint32_t* __restrict__ low,
                             const uint32_t* __restrict__ mapped, const uint32_t* __restrict__ r, uint32_t n) {
  const Fr lo = Fr::load_nc(low);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    Fr t = fe_add(fe_from_u32<FrParams>(i), lo);
    if (mapped) t = fe_add(t, fe_mul(Fr::load_nc(mapped + (uint64_t)i * 8), Fr::load_nc(r)));
    t.store(T + (uint64_t)i * 8);
  }
}

// The histogram and A = 1 / (S + beta) in one pass.  Every query equals a table entry T[idx], so
// A_i = B[idx] is a gather from the table's inverses (2 MB, cache-resident) instead of a batched
// inversion over the queries.  i runs over the PADDED layout (sub-rows of inner_pad columns of which
// the first `inner` come from src, the rest are padding = table entry pad_bin, counted separately).
// A query outside the table sets the status bit (the prover then fails) and gets A = 0.
__global__ void k_hist_gather(const uint32_t* __restrict__ src, uint64_t n_padded, uint32_t inner, uint32_t inner_pad,
                              const uint32_t* __restrict__ low, uint32_t pad_bin, const uint32_t* __restrict__ B,
                              uint32_t* __restrict__ A, uint32_t* __restrict__ hist, uint32_t n_bins,
                              uint32_t* __restrict__ status, uint32_t* __restrict__ idx_out) {
  const Fr lo = Fr::load_nc(low);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_padded; i += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t s = i;
    bool is_pad = false;
    if (inner) {
      const uint64_t row = i / inner_pad;
      const uint32_t col = (uint32_t)(i - row * inner_pad);
      is_pad = col >= inner;
      s = row * inner + col;
    }
    uint32_t idx = pad_bin;
    bool ok = true;
    if (!is_pad) {
      Fr d = fe_from_mont(fe_sub(Fr::load_nc(src + s * 8), lo));
      uint32_t hi = d.v[1] | d.v[2] | d.v[3] | d.v[4] | d.v[5] | d.v[6] | d.v[7];
      ok = hi == 0 && d.v[0] < n_bins;
      idx = d.v[0];
      if (ok) atomicAdd(hist + idx, 1u);
      else atomicOr(status, STATUS_HIST_RANGE);
    }
    Fr a = ok ? Fr::load_nc(B + (uint64_t)idx * 8) : Fr::zero();
    a.store(A + i * 8);
    if (idx_out) idx_out[i] = (is_pad || !ok) ? 0xFFFFFFFFu : idx;  // table entry per element, padding left out
  }
}

__global__ void k_hist_add(uint32_t* hist, uint32_t bin, uint32_t count) {
  if (threadIdx.x == 0 && blockIdx.x == 0) hist[bin] += count;
}

// S = S_in + r * S_out
__global__ void k_combine_pairs(const uint32_t* __restrict__ s_in, const uint32_t* __restrict__ s_out,
                                const uint32_t* __restrict__ r, uint32_t* __restrict__ out, uint64_t n) {
  const Fr rr = Fr::load_nc(r);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    fe_add(Fr::load_nc(s_in + i * 8), fe_mul(rr, Fr::load_nc(s_out + i * 8))).store(out + i * 8);
}

// partial[block] = sum_i a[i] * b[i]
__global__ void __launch_bounds__(LT) k_dot(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, uint64_t n,
                                            uint32_t* __restrict__ partial) {
  Fr acc[1] = {Fr::zero()};
  for (uint64_t i = (uint64_t)blockIdx.x * LT + threadIdx.x; i < n; i += (uint64_t)gridDim.x * LT)
    acc[0] = fe_add(acc[0], fe_mul(Fr::load_nc(a + i * 8), Fr::load_nc(b + i * 8)));
  lk_block_reduce_store<1>(acc, partial + (uint64_t)blockIdx.x * 8);
}

struct HalfWeights {
  const uint32_t* whi;
  const uint32_t* wlo;
  uint32_t lo_bits;
};
__device__ __forceinline__ Fr half_weight(const HalfWeights& hw, uint64_t g) {
  const uint64_t mask = (uint64_t(1) << hw.lo_bits) - 1;
  return fe_mul(Fr::load_nc(hw.whi + (g >> hw.lo_bits) * 8), Fr::load_nc(hw.wlo + (g & mask) * 8));
}

// Coefficients of (X0 + t dX)(Y0 + shift + t dY) weighted by w, accumulated into acc[0..2].
__device__ __forceinline__ void acc_product(Fr (&acc)[11], int base, const Fr& wX0, const Fr& wdX, const Fr& Y0s,
                                            const Fr& dY) {
  Fr c0 = fe_mul(wX0, Y0s);
  Fr c2 = fe_mul(wdX, dY);
  Fr mid = fe_mul(fe_add(wX0, wdX), fe_add(Y0s, dY));
  acc[base] = fe_add(acc[base], c0);
  acc[base + 1] = fe_add(acc[base + 1], fe_sub(fe_sub(mid, c0), c2));
  acc[base + 2] = fe_add(acc[base + 2], c2);
}

// Phase 1 round (reference: tLookup_phase1_step_poly + the two folds, src/tlookup.cu:117-151,233-238):
// sums 0..2 = sum_g w(g) * coefficients of A(t)(S(t)+beta); 3 = sum A0; 4 = sum dA; then fold A, S by v.
__global__ void __launch_bounds__(LT)
k_lookup_phase1(uint32_t* __restrict__ A, uint32_t* __restrict__ S, uint64_t half, const uint32_t* __restrict__ beta,
                const uint32_t* __restrict__ v, HalfWeights hw, uint32_t* __restrict__ partial) {
  const Fr bb = Fr::load_nc(beta), vv = Fr::load_nc(v);
  Fr acc[11];
#pragma unroll
  for (int s = 0; s < 11; s++) acc[s] = Fr::zero();
  for (uint64_t g = (uint64_t)blockIdx.x * LT + threadIdx.x; g < half; g += (uint64_t)gridDim.x * LT) {
    Fr A0 = Fr::load(A + g * 8), S0 = Fr::load(S + g * 8);
    Fr dA = fe_sub(Fr::load(A + (g + half) * 8), A0);
    Fr dS = fe_sub(Fr::load(S + (g + half) * 8), S0);
    fe_add(A0, fe_mul(vv, dA)).store(A + g * 8);
    fe_add(S0, fe_mul(vv, dS)).store(S + g * 8);
    Fr w = half_weight(hw, g);
    acc_product(acc, 0, fe_mul(w, A0), fe_mul(w, dA), fe_add(S0, bb), dS);
    acc[3] = fe_add(acc[3], A0);
    acc[4] = fe_add(acc[4], dA);
  }
  Fr out[5] = {acc[0], acc[1], acc[2], acc[3], acc[4]};
  lk_block_reduce_store<5>(out, partial + (uint64_t)blockIdx.x * 5 * 8);
}

// Phase 2 round (reference: tLookup_phase2_step_poly + tLookup_phase2_reduce_kernel, src/tlookup.cu:153-214):
// sums 0..2 weighted A(t)(S(t)+beta); 3..5 weighted B(t)(T(t)+beta); 6 sum A0; 7 sum dA; 8..10 m(t)B(t);
// then fold A, S, B, T, m by v.
__global__ void __launch_bounds__(LT)
k_lookup_phase2(uint32_t* __restrict__ A, uint32_t* __restrict__ S, uint32_t* __restrict__ B, uint32_t* __restrict__ T,
                uint32_t* __restrict__ M, uint64_t half, const uint32_t* __restrict__ beta,
                const uint32_t* __restrict__ v, HalfWeights hw, uint32_t* __restrict__ partial) {
  const Fr bb = Fr::load_nc(beta), vv = Fr::load_nc(v);
  Fr acc[11];
#pragma unroll
  for (int s = 0; s < 11; s++) acc[s] = Fr::zero();
  for (uint64_t g = (uint64_t)blockIdx.x * LT + threadIdx.x; g < half; g += (uint64_t)gridDim.x * LT) {
    Fr w = half_weight(hw, g);
    {
      Fr A0 = Fr::load(A + g * 8), S0 = Fr::load(S + g * 8);
      Fr dA = fe_sub(Fr::load(A + (g + half) * 8), A0);
      Fr dS = fe_sub(Fr::load(S + (g + half) * 8), S0);
      fe_add(A0, fe_mul(vv, dA)).store(A + g * 8);
      fe_add(S0, fe_mul(vv, dS)).store(S + g * 8);
      acc_product(acc, 0, fe_mul(w, A0), fe_mul(w, dA), fe_add(S0, bb), dS);
      acc[6] = fe_add(acc[6], A0);
      acc[7] = fe_add(acc[7], dA);
    }
    Fr B0 = Fr::load(B + g * 8), T0 = Fr::load(T + g * 8), M0 = Fr::load(M + g * 8);
    Fr dB = fe_sub(Fr::load(B + (g + half) * 8), B0);
    Fr dT = fe_sub(Fr::load(T + (g + half) * 8), T0);
    Fr dM = fe_sub(Fr::load(M + (g + half) * 8), M0);
    fe_add(B0, fe_mul(vv, dB)).store(B + g * 8);
    fe_add(T0, fe_mul(vv, dT)).store(T + g * 8);
    fe_add(M0, fe_mul(vv, dM)).store(M + g * 8);
    acc_product(acc, 3, fe_mul(w, B0), fe_mul(w, dB), fe_add(T0, bb), dT);
    acc_product(acc, 8, M0, dM, B0, dB);
  }
  lk_block_reduce_store<11>(acc, partial + (uint64_t)blockIdx.x * 11 * 8);
}

static uint32_t lk_blocks(const grape_ctx* ctx, uint64_t n) {
  uint64_t b = (n + LT - 1) / LT;
  uint64_t cap = (uint64_t)ctx->sm_count * 8;
  return (uint32_t)std::max<uint64_t>(std::min(b, cap), 1);
}

static int upload(grape_ctx* ctx, const HostFr* h, size_t n, uint32_t** d) {
  int rc = arena_alloc_t(ctx, n * 8 + 8, d);
  if (rc) return rc;
  if (n) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(*d, h, n * 32, cudaMemcpyHostToDevice, ctx->stream));
  return GRAPE_OK;
}

struct P4 {
  HostFr c[4];
};
static HostFr p4_at01(const P4& p) {
  HostFr s = p.c[0];
  for (int i = 0; i < 4; i++) s = fr_add(s, p.c[i]);
  return s;
}
static HostFr p4_eval(const P4& p, const HostFr& x) {
  HostFr acc = p.c[3];
  for (int i = 2; i >= 0; i--) acc = fr_add(fr_mul(acc, x), p.c[i]);
  return acc;
}
// (q0 + q1 t + q2 t^2) * ((1-u) + (2u-1) t)
static P4 mul_eq(const HostFr q[3], const HostFr& u) {
  HostFr e0 = fr_sub(fr_one(), u), e1 = fr_sub(fr_add(u, u), fr_one());
  P4 p;
  p.c[0] = fr_mul(q[0], e0);
  p.c[1] = fr_add(fr_mul(q[1], e0), fr_mul(q[0], e1));
  p.c[2] = fr_add(fr_mul(q[2], e0), fr_mul(q[1], e1));
  p.c[3] = fr_mul(q[2], e1);
  return p;
}

}  // namespace grape

using namespace grape;


static int lookup_create(grape_ctx* ctx, int32_t low, uint32_t len, const int32_t* d_map, grape_lookup** out) {
  if (!ctx || !out) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (len == 0) return fail(ctx, GRAPE_ERR_INVALID, "lookup: empty table");
  const uint32_t n = 1u << log2ceil(len);
  if (d_map && n != len) return fail(ctx, GRAPE_ERR_INVALID, "lookup: a mapping table must have a power-of-two length");
  grape_lookup* lk = new grape_lookup();
  lk->ctx = ctx;
  lk->low = low;
  lk->n = n;
  lk->mapping = d_map != nullptr;
  lk->alpha = rng_draw_fr(ctx->rng);               // reference: tLookup ctor, src/tlookup.cu:247
  if (lk->mapping) lk->r = rng_draw_fr(ctx->rng);  // reference: src/tlookup.cu:351
  lk->beta = fr_from_u64(n);
  const size_t bytes = (size_t)n * 32;
  if (cudaMalloc(&lk->T, bytes) != cudaSuccess || cudaMalloc(&lk->B, bytes) != cudaSuccess ||
      cudaMalloc(&lk->m, bytes) != cudaSuccess || cudaMalloc(&lk->hist, (size_t)n * 4) != cudaSuccess ||
      (lk->mapping && cudaMalloc(&lk->mapped, bytes) != cudaSuccess)) {
    cudaGetLastError();
    grape_lookup_destroy(lk);
    return fail(ctx, GRAPE_ERR_NOMEM, "lookup: table allocation failed");
  }
  arena_reset(ctx);
  HostFr consts[3] = {fr_from_i64(low), lk->beta, lk->r};
  uint32_t* d_c;
  int rc = upload(ctx, consts, 3, &d_c);
  if (rc) {
    grape_lookup_destroy(lk);
    return rc;
  }
  if (lk->mapping) {
    rc = grape_fr_from_i32(ctx, d_map, lk->mapped, n);
    if (rc) {
      grape_lookup_destroy(lk);
      return rc;
    }
  }
  cudaMemsetAsync(lk->m, 0, bytes, ctx->stream);
  k_table_init<<<lk_blocks(ctx, n), LT, 0, ctx->stream>>>(lk->T, d_c, lk->mapped, d_c + 16, n);
  ctx->launches += 1;
  // B = 1 / (T + beta), batched
  rc = fr_inverse_async(ctx, lk->T, d_c + 8, lk->B, n);
  if (rc == GRAPE_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess)
    rc = fail(ctx, GRAPE_ERR_CUDA, "lookup: table set-up failed on the device");
  if (rc) {
    grape_lookup_destroy(lk);
    return rc;
  }
  *out = lk;
  return GRAPE_OK;
}

extern "C" int grape_lookup_range_create(grape_ctx* ctx, int32_t low, uint32_t len, grape_lookup** out) {
  if (ctx) grape::make_device_current(ctx);
  return lookup_create(ctx, low, len, nullptr, out);
}

extern "C" int grape_lookup_mapping_create(grape_ctx* ctx, int32_t low, uint32_t len, const int32_t* d_map,
                                           grape_lookup** out) {
  if (ctx) grape::make_device_current(ctx);
  if (!d_map) return fail(ctx, GRAPE_ERR_INVALID, "lookup: null mapping table");
  return lookup_create(ctx, low, len, d_map, out);
}

extern "C" int grape_lookup_destroy(grape_lookup* lk) {
  if (!lk) return GRAPE_OK;
  if (lk->ctx) cudaStreamSynchronize(lk->ctx->stream);
  cudaFree(lk->T);
  cudaFree(lk->B);
  cudaFree(lk->m);
  cudaFree(lk->hist);
  cudaFree(lk->mapped);
  if (lk->ev_commit0) {
    cudaEventDestroy(lk->ev_commit0);
    cudaEventDestroy(lk->ev_commit1);
  }
  delete lk;
  return GRAPE_OK;
}

extern "C" int grape_lookup_params(const grape_lookup* lk, void* h_alpha, void* h_beta, void* h_r, uint32_t* n) {
  if (!lk) return GRAPE_ERR_INVALID;
  if (h_alpha) memcpy(h_alpha, &lk->alpha, 32);
  if (h_beta) memcpy(h_beta, &lk->beta, 32);
  if (h_r) memcpy(h_r, &lk->r, 32);
  if (n) *n = lk->n;
  return GRAPE_OK;
}

extern "C" int grape_lookup_last_proof(const grape_lookup* lk, void* h_finals, void* h_u, uint32_t u_capacity,
                                       uint32_t* n_u) {
  if (!lk || !lk->has_last) return GRAPE_ERR_INVALID;
  if (h_finals) memcpy(h_finals, lk->last_finals, sizeof lk->last_finals);
  if (n_u) *n_u = (uint32_t)lk->last_u.size();
  if (h_u) {
    if (u_capacity < lk->last_u.size()) return GRAPE_ERR_LIMIT;
    memcpy(h_u, lk->last_u.data(), lk->last_u.size() * 32);
  }
  return GRAPE_OK;
}

extern "C" int grape_lookup_last_commit_seconds(const grape_lookup* lk, double* seconds) {
  if (!lk || !seconds) return GRAPE_ERR_INVALID;
  *seconds = lk->last_commit_ms * 1e-3;
  return GRAPE_OK;
}

extern "C" const void* grape_lookup_table(const grape_lookup* lk, int which) {
  if (!lk) return nullptr;
  return which == 0 ? lk->T : which == 1 ? lk->B : which == 2 ? lk->m : lk->mapped;
}

// Multiplicities of the queries d_S (D Fr elements) into lk->m; pad_count is added to the bin of
// value zero (reference: prep, src/tlookup.cu:265-286).
// The prover proper.  d_S: queries (D elements, buffer of Dpad = 2^ceil(log2 D) elements when padding
// applies), consumed; d_A: buffer of Dpad elements that receives 1/(S+beta) and is consumed.
static int lookup_prove(grape_ctx* ctx, grape_lookup* lk, uint32_t* d_S, uint64_t D, uint32_t* d_A,
                        const HostFr* v, uint32_t n_v, uint32_t inner, uint32_t inner_pad, const HostFr& pad_value,
                        const grape_table* table, uint32_t msm_size, void* d_com_A, void* d_com_m,
                        HostFr* h_claim, HostFr* h_transcript, uint32_t transcript_capacity, uint32_t* n_rounds,
                        const uint32_t* d_hist_src) {
  const uint32_t N = lk->n, lN = log2ceil(N);
  const uint32_t lD = log2ceil(D);
  const uint64_t Dp = uint64_t(1) << lD;
  if (n_v != lD) return fail(ctx, GRAPE_ERR_INVALID, "lookup: v.size() != ceilLog2(D)");
  if (table && table->curve != 0) return fail(ctx, GRAPE_ERR_INVALID, "lookup: commitments are built over BN254 only");
  if (Dp < N) return fail(ctx, GRAPE_ERR_INVALID, "lookup: fewer queries than table entries is not supported");
  if (D != Dp && (inner == 0 || inner_pad < inner || D % inner != 0 || (D / inner) * (uint64_t)inner_pad != Dp))
    return fail(ctx, GRAPE_ERR_INVALID, "lookup: cannot pad the queries to a power of two with the given row lengths");
  // u is drawn before anything else, as in the reference (src/tlookup.cu:293)
  std::vector<HostFr> u(lD);
  for (auto& x : u) x = rng_draw_fr(ctx->rng);
  uint32_t *d_u, *d_v, *d_c;
  int rc;
  if ((rc = upload(ctx, u.data(), lD, &d_u))) return rc;
  if ((rc = upload(ctx, v, lD, &d_v))) return rc;
  HostFr consts[3] = {fr_from_i64(lk->low), lk->beta, pad_value};
  if ((rc = upload(ctx, consts, 3, &d_c))) return rc;
  // multiplicities, and A = 1 / (S + beta) gathered from the table's inverses in the same pass
  // (reference: prep + the inversion of S + beta, src/tlookup.cu:250-262,296-318)
  const int64_t pad_bin = -(int64_t)lk->low;
  if (D != Dp && (pad_bin < 0 || pad_bin >= (int64_t)N))
    return fail(ctx, GRAPE_ERR_INVALID, "lookup: padding needs 0 inside the table range");
  // Commit A by the bucket method?  Cost per row in units of one mixed addition of the direct kernel:
  // direct = elements * windows of the table; bucketed = 1.2 * elements (stage 1: one addition per
  // element, some spread inside a warp) + 40 * table entries as MEASURED (64 rows of 2^18 elements over a
  // 2^16-entry table: 0.53 ms per row against 0.89 ms; on paper 1.3 for the normalisation + 20 windows *
  // (1.08 for the bucket sums + 0.19 for the running sums) = 27, the rest is lanes idle at slice ends).
  uint32_t* d_idx = nullptr;
  if (table && msm_size && ctx->bucket_mode != 0 && N % 32 == 0) {
    const uint64_t a_wd0 = (uint64_t)msm_size * GRAPE_COM_SCALE;
    const uint64_t valid = (D != Dp && a_wd0 % inner_pad == 0) ? a_wd0 / inner_pad * inner : a_wd0;
    const double direct = (double)valid * ((254 + table->window_bits - 1) / table->window_bits);
    const double bucketed = 1.2 * (double)valid + 40.0 * N;
    if (ctx->bucket_mode == 2 || bucketed < 0.9 * direct) {
      if ((rc = arena_alloc_t(ctx, (size_t)Dp, &d_idx))) return rc;
    }
  }
  GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(lk->hist, 0, (size_t)N * 4, ctx->stream));
  if (D == Dp) {
    k_hist_gather<<<lk_blocks(ctx, Dp), LT, 0, ctx->stream>>>(d_hist_src, Dp, 0, 0, d_c, 0, lk->B, d_A, lk->hist, N,
                                                              ctx->d_status, d_idx);
    ctx->launches += 1;
  } else {
    // row-pad inner -> inner_pad (like FrTensor::pad): the padded S is built in a scratch buffer because
    // both d_S (dense) and d_A (gather target) are live until the gather has read the dense queries
    uint32_t* padded = nullptr;
    if ((rc = arena_alloc_t(ctx, (size_t)Dp * 8, &padded))) return rc;
    if ((rc = grape_fr_pad(ctx, d_S, padded, inner, inner_pad, Dp, d_c + 16))) return rc;
    k_hist_gather<<<lk_blocks(ctx, Dp), LT, 0, ctx->stream>>>(d_hist_src, Dp, inner, inner_pad, d_c, (uint32_t)pad_bin,
                                                              lk->B, d_A, lk->hist, N, ctx->d_status, d_idx);
    k_hist_add<<<1, 32, 0, ctx->stream>>>(lk->hist, (uint32_t)pad_bin, (uint32_t)(Dp - D));
    ctx->launches += 2;
    GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_S, padded, Dp * 32, cudaMemcpyDeviceToDevice, ctx->stream));
  }
  if ((rc = grape_fr_from_u32(ctx, lk->hist, lk->m, N))) return rc;
  // commitments to A and m (reference: src/tlookup.cu:319-323); optional here
  lk->last_commit_ms = 0.f;
  if (table) {
    if (!lk->ev_commit0) {
      GRAPE_CUDA_TRY(ctx, cudaEventCreate(&lk->ev_commit0));
      GRAPE_CUDA_TRY(ctx, cudaEventCreate(&lk->ev_commit1));
    }
    GRAPE_CUDA_TRY(ctx, cudaEventRecord(lk->ev_commit0, ctx->stream));
    if (msm_size == 0 || Dp % ((uint64_t)msm_size * GRAPE_COM_SCALE) != 0)
      return fail(ctx, GRAPE_ERR_INVALID, "lookup: D must be a multiple of msm_size * 16");
    const uint32_t m_wd = (1u << (lN / 2)) * GRAPE_COM_SCALE;
    if (N % m_wd != 0 || N < m_wd) return fail(ctx, GRAPE_ERR_INVALID, "lookup: table too small to commit its multiplicities");
    void* tmp = nullptr;
    if (!d_com_A) {
      if ((rc = arena_alloc(ctx, (Dp / ((uint64_t)msm_size * GRAPE_COM_SCALE)) * 96, &tmp))) return rc;
      d_com_A = tmp;
    }
    if (!d_com_m) {
      if ((rc = arena_alloc(ctx, (size_t)(N / m_wd) * 96, &tmp))) return rc;
      d_com_m = tmp;
    }
    const uint32_t a_wd = msm_size * GRAPE_COM_SCALE;
    bool committed = false;
    if (d_idx) {
      // bucket method; the padded columns (left out of d_idx) still contribute their shared point
      uint32_t* extra = nullptr;
      if (D != Dp) {
        if (a_wd % inner_pad == 0) {
          if ((rc = constant_columns_point_async(ctx, table, a_wd, inner, inner_pad, d_A + (size_t)inner * 8, &extra)))
            return rc;
        } else {
          d_idx = nullptr;  // rows do not consist of whole padded sub-rows: commit directly
        }
      }
      if (d_idx) {
        rc = commit_gathered_async(ctx, table, d_idx, lk->B, N, Dp, a_wd, extra, d_com_A);
        if (rc == GRAPE_OK) committed = true;
        else if (rc != GRAPE_ERR_INVALID) return rc;  // INVALID: shape not supported, fall through
      }
    }
    if (committed) {
    } else if (D != Dp && a_wd % inner_pad == 0) {
      // the padded columns of every row hold the same value 1 / (pad + beta): element `inner` of A is one of them
      if ((rc = commit_fr_padded_async(ctx, table, d_A, Dp, a_wd, inner, inner_pad, d_A + (size_t)inner * 8, d_com_A)))
        return rc;
    } else if ((rc = commit_fr_async(ctx, table, d_A, Dp, a_wd, d_com_A))) {
      return rc;
    }
    if ((rc = commit_fr_async(ctx, table, lk->m, N, m_wd, d_com_m))) return rc;
    GRAPE_CUDA_TRY(ctx, cudaEventRecord(lk->ev_commit1, ctx->stream));
  }
  // working copies of B, T, m (the rounds fold in place), sum_j B_j m_j
  uint32_t *Bw, *Tw, *Mw, *partial, *sums, *whi, *wlo, *d_bm;
  if ((rc = arena_alloc_t(ctx, (size_t)N * 8, &Bw))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)N * 8, &Tw))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)N * 8, &Mw))) return rc;
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(Bw, lk->B, (size_t)N * 32, cudaMemcpyDeviceToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(Tw, lk->T, (size_t)N * 32, cudaMemcpyDeviceToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(Mw, lk->m, (size_t)N * 32, cudaMemcpyDeviceToDevice, ctx->stream));
  const uint32_t max_blocks = ctx->sm_count * 8;
  if ((rc = arena_alloc_t(ctx, (size_t)max_blocks * 11 * 8 + 64, &partial))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)(lD + 2) * 11 * 8, &sums))) return rc;
  const uint32_t lo_cap = (lD + 1) / 2, hi_cap = lD - lo_cap;
  if ((rc = arena_alloc_t(ctx, ((size_t)1 << hi_cap) * 8 + 8, &whi))) return rc;
  if ((rc = arena_alloc_t(ctx, ((size_t)1 << lo_cap) * 8 + 8, &wlo))) return rc;
  if ((rc = arena_alloc_t(ctx, 8 + 8, &d_bm))) return rc;
  {
    uint32_t blocks = lk_blocks(ctx, N);
    k_dot<<<blocks, LT, 0, ctx->stream>>>(Bw, Mw, N, partial);
    k_lk_reduce<1><<<1, LT, 0, ctx->stream>>>(partial, blocks, d_bm);
    ctx->launches += 2;
  }
  // rounds: phase 1 consumes v[lN..) top down, phase 2 consumes v[..lN) top down; u is consumed from its top
  uint64_t cur = Dp;
  uint32_t round = 0;
  const uint32_t n_phase1 = lD - lN;
  for (uint32_t i = 0; i < lD; i++, round++) {
    const uint64_t half = cur / 2;
    const uint32_t rem = lD - i - 1;  // variables of the weights: u[0 .. rem)
    const uint32_t lo_bits = std::min(rem, lo_cap), hi_bits = rem - lo_bits;
    eq_weights_async(ctx, d_u, lo_bits, 1u << lo_bits, wlo);
    eq_weights_async(ctx, d_u + (size_t)lo_bits * 8, hi_bits, 1u << hi_bits, whi);
    HalfWeights hw{whi, wlo, lo_bits};
    const uint32_t* dv = d_v + (size_t)(lD - i - 1) * 8;  // phase 1: v1.back() = v[lD-1-i]; phase 2 continues downwards
    const uint32_t blocks = lk_blocks(ctx, half);
    if (i < n_phase1) {
      k_lookup_phase1<<<blocks, LT, 0, ctx->stream>>>(d_A, d_S, half, d_c + 8, dv, hw, partial);
      k_lk_reduce<5><<<1, LT, 0, ctx->stream>>>(partial, blocks, sums + (size_t)round * 11 * 8);
    } else {
      k_lookup_phase2<<<blocks, LT, 0, ctx->stream>>>(d_A, d_S, Bw, Tw, Mw, half, d_c + 8, dv, hw, partial);
      k_lk_reduce<11><<<1, LT, 0, ctx->stream>>>(partial, blocks, sums + (size_t)round * 11 * 8);
    }
    ctx->launches += 2;
    cur = half;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  std::vector<HostFr> hs((size_t)lD * 11 + 2);
  if (lD) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(hs.data(), sums, (size_t)lD * 11 * 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&hs[(size_t)lD * 11], d_bm, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&hs[(size_t)lD * 11 + 1], d_S, 32, cudaMemcpyDeviceToHost, ctx->stream));
  lk->has_last = false;
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&lk->last_finals[0], d_A, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&lk->last_finals[1], d_S, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&lk->last_finals[2], Bw, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&lk->last_finals[3], Tw, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&lk->last_finals[4], Mw, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  lk->last_u = u;
  if (table) cudaEventElapsedTime(&lk->last_commit_ms, lk->ev_commit0, lk->ev_commit1);
  uint32_t st = 0;
  GRAPE_CUDA_TRY(ctx, cudaMemcpy(&st, ctx->d_status, 4, cudaMemcpyDeviceToHost));
  if (st & STATUS_HIST_RANGE) {
    cudaMemsetAsync(ctx->d_status, 0, 4, ctx->stream);
    return fail(ctx, GRAPE_ERR_CHECK, "lookup: a query lies outside the table");
  }
  // host pass (reference: tLookup_phase1 / tLookup_phase2 recursion)
  HostFr alpha = lk->alpha, alpha_sq = fr_mul(alpha, alpha);
  HostFr C = fr_sub(alpha_sq, hs[(size_t)lD * 11]);
  HostFr claim = fr_add(alpha, alpha_sq);
  const HostFr two_inv = fr_inv(fr_from_u64(2));
  const HostFr ratio = fr_mul(fr_from_u64(N), fr_inv(fr_from_u64(Dp)));
  uint32_t emitted = 0;
  for (uint32_t i = 0; i < lD; i++) {
    const HostFr* s = &hs[(size_t)i * 11];
    const HostFr u_top = u[lD - i - 1], v_now = v[lD - i - 1];
    P4 p;
    if (i < n_phase1) {
      HostFr q[3] = {fr_mul(s[0], alpha), fr_mul(s[1], alpha), fr_mul(s[2], alpha)};
      p = mul_eq(q, u_top);
      p.c[0] = fr_add(fr_add(p.c[0], s[3]), fr_mul(C, two_inv));
      p.c[1] = fr_add(p.c[1], s[4]);
    } else {
      const HostFr coef = fr_mul(ratio, alpha_sq);
      HostFr q[3];
      for (int k = 0; k < 3; k++) q[k] = fr_add(fr_mul(s[k], alpha), fr_mul(s[3 + k], coef));
      p = mul_eq(q, u_top);
      p.c[0] = fr_add(p.c[0], s[6]);
      p.c[1] = fr_add(p.c[1], s[7]);
      for (int k = 0; k < 3; k++) p.c[k] = fr_sub(p.c[k], fr_mul(s[8 + k], ratio));
    }
    if (h_transcript && emitted < transcript_capacity) memcpy(h_transcript + (size_t)emitted * 4, p.c, 128);
    emitted++;
    if (p4_at01(p) != claim)
      return fail(ctx, GRAPE_ERR_CHECK, std::string(i < n_phase1 ? "tLookup_phase1" : "tLookup_phase2") +
                                            ": claim != p(0) + p(1) in round " + std::to_string(i));
    claim = p4_eval(p, v_now);
    const HostFr e = fr_eq2(u_top, v_now);
    alpha = fr_mul(alpha, e);
    if (i < n_phase1) C = fr_mul(C, two_inv);
    else alpha_sq = fr_mul(alpha_sq, e);
  }
  if (n_rounds) *n_rounds = emitted;
  *h_claim = hs[(size_t)lD * 11 + 1];
  lk->has_last = true;
  return GRAPE_OK;
}

// tLookupRange::prove (src/tlookup.cu:288-343).
extern "C" int grape_lookup_prove_range(grape_ctx* ctx, grape_lookup* lk, void* d_S, uint64_t D, void* d_A,
                                        const void* h_v, uint32_t n_v, uint32_t inner, uint32_t inner_pad,
                                        const grape_table* table, uint32_t msm_size, void* d_com_A, void* d_com_m,
                                        void* h_claim, void* h_transcript, uint32_t transcript_capacity,
                                        uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !lk || !d_S || !d_A || !h_v || !h_claim) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (lk->mapping) return fail(ctx, GRAPE_ERR_INVALID, "lookup: use grape_lookup_prove_mapping for a mapping table");
  arena_reset(ctx);
  return lookup_prove(ctx, lk, (uint32_t*)d_S, D, (uint32_t*)d_A, (const HostFr*)h_v, n_v, inner, inner_pad, fr_zero(),
                      table, msm_size, d_com_A, d_com_m, (HostFr*)h_claim, (HostFr*)h_transcript, transcript_capacity,
                      n_rounds, (const uint32_t*)d_S);
}

// tLookupRangeMapping::prove (src/tlookup.cu:398-456): queries are pairs (S_in, S_out = f(S_in)).
// d_S_work: buffer of 2^ceil(log2 D) elements that receives S_in + r*S_out and is consumed.
extern "C" int grape_lookup_prove_mapping(grape_ctx* ctx, grape_lookup* lk, const void* d_S_in, const void* d_S_out,
                                          uint64_t D, void* d_S_work, void* d_A, const void* h_v, uint32_t n_v,
                                          uint32_t inner, uint32_t inner_pad, const grape_table* table,
                                          uint32_t msm_size, void* d_com_A, void* d_com_m, void* h_claim,
                                          void* h_transcript, uint32_t transcript_capacity, uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !lk || !d_S_in || !d_S_out || !d_S_work || !d_A || !h_v || !h_claim)
    return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (!lk->mapping) return fail(ctx, GRAPE_ERR_INVALID, "lookup: not a mapping table");
  arena_reset(ctx);
  uint32_t* d_r;
  int rc = upload(ctx, &lk->r, 1, &d_r);
  if (rc) return rc;
  k_combine_pairs<<<lk_blocks(ctx, D), LT, 0, ctx->stream>>>((const uint32_t*)d_S_in, (const uint32_t*)d_S_out, d_r,
                                                             (uint32_t*)d_S_work, D);
  ctx->launches += 1;
  // pad value = map[-low] * r (reference: src/tlookup.cu:415)
  HostFr pad_value = fr_zero();
  if (D != (uint64_t(1) << log2ceil(D))) {
    int64_t bin = -(int64_t)lk->low;
    if (bin < 0 || bin >= (int64_t)lk->n) return fail(ctx, GRAPE_ERR_INVALID, "lookup: padding needs 0 inside the table range");
    HostFr mv;
    GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&mv, lk->mapped + (size_t)bin * 8, 32, cudaMemcpyDeviceToHost, ctx->stream));
    GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    pad_value = fr_mul(mv, lk->r);
  }
  return lookup_prove(ctx, lk, (uint32_t*)d_S_work, D, (uint32_t*)d_A, (const HostFr*)h_v, n_v, inner, inner_pad,
                      pad_value, table, msm_size, d_com_A, d_com_m, (HostFr*)h_claim, (HostFr*)h_transcript,
                      transcript_capacity, n_rounds, (const uint32_t*)d_S_in);
}
