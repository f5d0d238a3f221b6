// Row commitments of a GATHERED tensor by the bucket method.
//
// The lookup argument commits A with A_i = B[idx_i]: every element is one of the n_bins values of
// the table's inverse vector B (src/tlookup.cu:296-323 forms A = 1/(S+beta) element by element and
// commits it with 32 additions per element).  When a commitment row holds several times more
// elements than the table has entries, most of those additions are redundant:
//
//   C_row = sum_i B[idx_i] * G_i = sum_t B[t] * P_t,      P_t = sum of the G_i of the row with idx_i = t.
//
//   stage 1  per row: counting sort of the row's elements by table entry in shared memory
//            (k_row_sort), then one thread per 8 consecutive entries adds the generators of each
//            entry and normalises the 8 sums with one shared inversion (k_bucket_points)
//            -- ONE addition per element;
//   stage 2  per row a variable-base multi-scalar multiplication of the n_bins points P_t by the
//            scalars B[t], which are the SAME for every row: their signed 13-bit digits are sorted
//            once per window (k_digit_keys + k_row_sort again), and one block per (row, window)
//            walks the magnitudes from the top with the running-sum rule, every thread taking a
//            contiguous range of magnitudes (k_window_sums) -- n_bins additions per window;
//   stage 3  the finalize kernel of the fixed-base path recombines the windows (Horner) and adds
//            the shared point of the padded columns.
//
// Cost per row: elements + n_bins * (windows + ~3) additions instead of elements * windows.  The
// result is the same group element, so the normalised record is bit-identical.
#include <algorithm>

#include "ctx.cuh"
#include "curve.cuh"

namespace grape {

// implemented in msm.cu
int finalize_bn254_async(grape_ctx* ctx, const Xyzz* partials, uint32_t n_chunks, uint32_t groups, uint32_t group_bits,
                         uint64_t rows, void* d_out, const void* d_extra);

constexpr int SORT_THREADS = 1024;
constexpr uint32_t SORT_PART_BINS = 32768;     // 128 KB of shared counters per block
constexpr uint32_t STAGE2_BITS = 13;           // window width of the variable-base stage
constexpr uint32_t STAGE2_HALF = 1u << (STAGE2_BITS - 1);
constexpr uint32_t STAGE2_WINDOWS = (254 + STAGE2_BITS - 1) / STAGE2_BITS;  // 20

// Counting sort of one row of keys (grid: rows x parts of the key space, each part's counters in
// shared memory).  keys: [rows][wd], a key >= n_bins (0xFFFFFFFF marks padding) is left out.
// offs: [rows][n_bins + 1] start of every key's run in `sorted`; sorted: [rows][wd] element positions.
__global__ void __launch_bounds__(SORT_THREADS) k_row_sort(const uint32_t* __restrict__ keys, uint32_t wd,
                                                           uint32_t n_bins, uint32_t* __restrict__ offs,
                                                           uint32_t* __restrict__ sorted) {
  extern __shared__ uint32_t cnt[];
  __shared__ uint32_t warp_tot[SORT_THREADS / 32];
  __shared__ uint32_t below_total;
  const uint64_t row = blockIdx.x;
  const uint32_t lo = blockIdx.y * SORT_PART_BINS;
  const uint32_t hi = min(n_bins, lo + SORT_PART_BINS);
  const uint32_t nb = hi - lo;
  const uint32_t tid = threadIdx.x;
  for (uint32_t b = tid; b < nb; b += SORT_THREADS) cnt[b] = 0;
  if (tid == 0) below_total = 0;
  __syncthreads();
  const uint32_t* r = keys + row * wd;
  uint32_t below = 0;
  for (uint32_t i = tid; i < wd; i += SORT_THREADS) {
    const uint32_t k = __ldg(r + i);
    if (k < lo) below++;
    else if (k < hi) atomicAdd(&cnt[k - lo], 1u);
  }
  for (int off = 16; off > 0; off >>= 1) below += __shfl_down_sync(0xffffffffu, below, off);
  if ((tid & 31) == 0 && below) atomicAdd(&below_total, below);
  __syncthreads();
  // exclusive scan: thread t owns `per` consecutive counters
  const uint32_t per = (nb + SORT_THREADS - 1) / SORT_THREADS;
  const uint32_t b0 = min(nb, tid * per), b1 = min(nb, b0 + per);
  uint32_t local = 0;
  for (uint32_t b = b0; b < b1; b++) local += cnt[b];
  uint32_t incl = local;
  for (int off = 1; off < 32; off <<= 1) {
    uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
    if ((tid & 31) >= (uint32_t)off) incl += v;
  }
  if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    uint32_t v = tid < SORT_THREADS / 32 ? warp_tot[tid] : 0, inc = v;
    for (int off = 1; off < 32; off <<= 1) {
      uint32_t u = __shfl_up_sync(0xffffffffu, inc, off);
      if (tid >= (uint32_t)off) inc += u;
    }
    warp_tot[tid] = inc - v;  // exclusive prefix of the warp totals
  }
  __syncthreads();
  uint32_t running = below_total + warp_tot[tid >> 5] + (incl - local);
  uint32_t* orow = offs + row * (uint64_t)(n_bins + 1);
  for (uint32_t b = b0; b < b1; b++) {
    const uint32_t c = cnt[b];
    orow[lo + b] = running;
    cnt[b] = running;  // becomes the scatter cursor
    running += c;
  }
  if (hi == n_bins && tid == SORT_THREADS - 1) orow[n_bins] = running;  // the last thread ends on the grand total
  __syncthreads();
  uint32_t* srow = sorted + row * wd;
  for (uint32_t i = tid; i < wd; i += SORT_THREADS) {
    const uint32_t k = __ldg(r + i);
    if (k >= lo && k < hi) srow[atomicAdd(&cnt[k - lo], 1u)] = i;
  }
}

// Stage 1 sums.  One thread: 8 consecutive table entries of one row; P[row][t] = sum of the
// generators of the row's elements with index t, affine ((0,0) when the entry does not occur).
constexpr int BUCKET_BATCH = 8;
__global__ void __launch_bounds__(128) k_bucket_points(const Affine* __restrict__ gens, const uint32_t* __restrict__ offs,
                                                       const uint32_t* __restrict__ sorted, uint32_t wd, uint32_t n_bins,
                                                       uint64_t n_threads, Affine* __restrict__ P) {
  const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= n_threads) return;
  const uint32_t per_row = n_bins / BUCKET_BATCH;
  const uint64_t row = gid / per_row;
  const uint32_t t0 = (uint32_t)(gid % per_row) * BUCKET_BATCH;
  const uint32_t* orow = offs + row * (uint64_t)(n_bins + 1);
  const uint32_t* srow = sorted + row * wd;
  Xyzz e[BUCKET_BATCH];
  Fp pref[BUCKET_BATCH];
  Fp run = Fp::one();
#pragma unroll 1
  for (int k = 0; k < BUCKET_BATCH; k++) {
    const uint32_t s = orow[t0 + k], en = orow[t0 + k + 1];
    Xyzz acc = Xyzz::inf();
#pragma unroll 1
    for (uint32_t j = s; j < en; j++) xyzz_madd(acc, Affine::load_nc(gens + srow[j]));
    e[k] = acc;
    Fp zp = acc.is_inf() ? Fp::one() : fe_mul(acc.zz, acc.zzz);
    run = fe_mul(run, zp);
    pref[k] = run;
  }
  Fp inv = fe_inv(run);
#pragma unroll 1
  for (int k = BUCKET_BATCH - 1; k >= 0; k--) {
    Fp zp = e[k].is_inf() ? Fp::one() : fe_mul(e[k].zz, e[k].zzz);
    Fp zinv = (k == 0) ? inv : fe_mul(inv, pref[k - 1]);
    inv = fe_mul(inv, zp);
    Affine out;
    if (e[k].is_inf()) {
      out = Affine::inf();
    } else {
      out.x = fe_mul(e[k].x, fe_mul(zinv, e[k].zzz));
      out.y = fe_mul(e[k].y, fe_mul(zinv, e[k].zz));
    }
    out.store(P + row * n_bins + t0 + k);
  }
}

// Signed digits of the n_bins scalars, window by window: mags[w][t] = |digit| (0 when the digit is
// zero: such an entry sorts to key 0, which stage 2 never visits), neg[w][t] = its sign.
struct Bias8 {
  uint32_t v[8];
};
__global__ void k_digit_keys(const uint32_t* __restrict__ B, uint32_t n_bins, Bias8 bias, uint32_t* __restrict__ mags,
                             uint8_t* __restrict__ neg) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_bins) return;
  Fr s = fe_from_mont(Fr::load_nc(B + (uint64_t)t * 8));
  uint32_t r[8];
  add8(r, s.v, bias.v);
  for (uint32_t w = 0; w < STAGE2_WINDOWS; w++) {
    const uint32_t bit = STAGE2_BITS * w, word = bit >> 5;
    const uint32_t lo = r[word], hi = word < 7 ? r[word + 1] : 0u;
    const uint32_t e = __funnelshift_r(lo, hi, bit & 31) & ((1u << STAGE2_BITS) - 1u);
    const int32_t d = (w + 1 == STAGE2_WINDOWS) ? (int32_t)e : (int32_t)e - (int32_t)STAGE2_HALF;
    mags[(uint64_t)w * n_bins + t] = d < 0 ? (uint32_t)(-d) : (uint32_t)d;
    neg[(uint64_t)w * n_bins + t] = d < 0 ? 1 : 0;
  }
}

// Stage 2.  One block per (row, window): sum over magnitudes m of m * (sum of the +-P_t whose digit
// has magnitude m).  Thread k takes the magnitudes (k*per, (k+1)*per] from the top down with the
// running-sum rule (run += bucket, tot += run), corrects by (k*per) * run, and the block adds up.
constexpr int WS_THREADS = 256;
__global__ void __launch_bounds__(WS_THREADS) k_window_sums(const Affine* __restrict__ P, uint32_t n_bins,
                                                            const uint32_t* __restrict__ offs2,
                                                            const uint32_t* __restrict__ sorted2,
                                                            const uint8_t* __restrict__ neg, Xyzz* __restrict__ partial) {
  __shared__ __align__(16) unsigned char red_raw[(WS_THREADS / 32) * sizeof(Xyzz)];
  Xyzz* red = reinterpret_cast<Xyzz*>(red_raw);
  const uint64_t row = blockIdx.x;
  const uint32_t w = blockIdx.y;
  const uint32_t tid = threadIdx.x;
  constexpr uint32_t per = STAGE2_HALF / WS_THREADS;
  const uint32_t base = tid * per;  // this thread's magnitudes are base + 1 .. base + per
  const uint32_t* o2 = offs2 + (uint64_t)w * (STAGE2_HALF + 2);
  const uint32_t* s2 = sorted2 + (uint64_t)w * n_bins;
  const uint8_t* ng = neg + (uint64_t)w * n_bins;
  const Affine* prow = P + row * n_bins;
  Xyzz run = Xyzz::inf(), tot = Xyzz::inf();
#pragma unroll 1
  for (uint32_t m = base + per; m > base; m--) {
    const uint32_t s = o2[m], en = o2[m + 1];
#pragma unroll 1
    for (uint32_t j = s; j < en; j++) {
      const uint32_t t = s2[j];
      Affine p = Affine::load_nc(prow + t);
      if (ng[t]) p.y = fe_neg(p.y);  // the point at infinity is (0, 0) and stays so
      xyzz_madd(run, p);
    }
    xyzz_add(tot, run);
  }
  // tot = sum (m - base) * bucket_m; add base * run by double-and-add over the bits of base
  if (base != 0 && !run.is_inf()) {
    Xyzz acc = Xyzz::inf();
#pragma unroll 1
    for (int bit = 31 - __clz(base); bit >= 0; bit--) {
      acc = xyzz_dbl(acc);
      if ((base >> bit) & 1u) xyzz_add(acc, run);
    }
    xyzz_add(tot, acc);
  }
#pragma unroll 1
  for (int off = 16; off > 0; off >>= 1) {
    Xyzz other = xyzz_shfl_down(tot, off);
    if ((tid & 31) < (uint32_t)off) xyzz_add(tot, other);
  }
  if ((tid & 31) == 0) tot.store(red + (tid >> 5));
  __syncthreads();
  if (tid == 0) {
    Xyzz acc = Xyzz::load(red);
#pragma unroll 1
    for (int k = 1; k < WS_THREADS / 32; k++) xyzz_add(acc, Xyzz::load(red + k));
    acc.store(partial + row * STAGE2_WINDOWS + w);
  }
}

// Row commitments  C_row = sum_i B[idx[row][i]] * G_i  (+ extra, the same point for every row).
//   d_idx: [size] table indices, 0xFFFFFFFF for elements that take no part; d_B: n_bins Fr scalars.
// Returns GRAPE_ERR_INVALID when the shape is not supported (the caller then commits directly).
int commit_gathered_async(grape_ctx* ctx, const grape_table* t, const uint32_t* d_idx, const uint32_t* d_B,
                          uint32_t n_bins, uint64_t size, uint32_t wd, const void* d_extra, void* d_out) {
  if (!t || t->curve != Bn254::ID || wd == 0 || wd > t->n_gens || size % wd != 0 || n_bins < BUCKET_BATCH ||
      n_bins % BUCKET_BATCH != 0 || n_bins > (1u << 24) || STAGE2_HALF % WS_THREADS != 0)
    return GRAPE_ERR_INVALID;
  const uint64_t rows = size / wd;
  if (rows == 0) return GRAPE_OK;
  if (rows > 0x7fffffffull) return GRAPE_ERR_INVALID;
  int rc;
  uint32_t *offs, *sorted, *mags, *offs2, *sorted2;
  uint8_t* neg;
  Affine* P;
  Xyzz* partial;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)(n_bins + 1), &offs))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)wd, &sorted))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)n_bins, &P))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &mags))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &neg))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * (STAGE2_HALF + 2), &offs2))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &sorted2))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * STAGE2_WINDOWS, &partial))) return rc;
  GRAPE_CUDA_TRY(ctx, cudaFuncSetAttribute(k_row_sort, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(SORT_PART_BINS * sizeof(uint32_t))));
  // stage 1
  {
    const uint32_t parts = (n_bins + SORT_PART_BINS - 1) / SORT_PART_BINS;
    const size_t smem = (size_t)std::min(n_bins, SORT_PART_BINS) * sizeof(uint32_t);
    k_row_sort<<<dim3((uint32_t)rows, parts), SORT_THREADS, smem, ctx->stream>>>(d_idx, wd, n_bins, offs, sorted);
    const Affine* gens = reinterpret_cast<const Affine*>(t->data) + (uint64_t)t->first_digit_row * t->n_gens;
    const uint64_t n_threads = rows * (n_bins / BUCKET_BATCH);
    k_bucket_points<<<(uint32_t)((n_threads + 127) / 128), 128, 0, ctx->stream>>>(gens, offs, sorted, wd, n_bins,
                                                                                   n_threads, P);
    ctx->launches += 2;
  }
  // stage 2: digits of the shared scalars, sorted by magnitude per window (keys 0 .. STAGE2_HALF)
  {
    Bias8 bias;
    for (int k = 0; k < 8; k++) bias.v[k] = 0;
    for (uint32_t w = 0; w + 1 < STAGE2_WINDOWS; w++) {
      const uint32_t bit = STAGE2_BITS * w + STAGE2_BITS - 1;
      bias.v[bit >> 5] |= 1u << (bit & 31);
    }
    k_digit_keys<<<(n_bins + 255) / 256, 256, 0, ctx->stream>>>(d_B, n_bins, bias, mags, neg);
    k_row_sort<<<dim3(STAGE2_WINDOWS, 1), SORT_THREADS, (STAGE2_HALF + 1) * sizeof(uint32_t), ctx->stream>>>(
        mags, n_bins, STAGE2_HALF + 1, offs2, sorted2);
    k_window_sums<<<dim3((uint32_t)rows, STAGE2_WINDOWS), WS_THREADS, 0, ctx->stream>>>(P, n_bins, offs2, sorted2, neg,
                                                                                        partial);
    ctx->launches += 3;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  // stage 3: Horner over the windows, extra point, normalisation
  return finalize_bn254_async(ctx, partial, 1, STAGE2_WINDOWS, STAGE2_BITS, rows, d_out, d_extra);
}

}  // namespace grape
