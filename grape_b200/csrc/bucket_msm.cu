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
//            (k_row_sort); one thread per 32 consecutive entries walks their elements in ONE flat loop
//            and stores the sum of every entry as it completes (k_bucket_sums) -- one addition per
//            element, lanes of a warp differ only by the spread of 32-entry totals; the sums are then
//            normalised to affine, 16 to an inversion (k_normalise);
//   stage 2  per row a variable-base multi-scalar multiplication of the n_bins points P_t by the
//            scalars B[t], which are the SAME for every row: their signed 13-bit digits are sorted
//            by magnitude once per window (k_digit_keys + k_row_sort + k_pack_entries).
//            2a (k_window_buckets): the sorted list of a window is cut into slices of about equal
//            length that end on magnitude boundaries; a lane walks one slice, adds the +-P_t of one
//            magnitude after the other and stores each magnitude's sum when it is complete.  Every
//            lane executes one mixed addition per step; a change of magnitude costs a store, not a
//            divergent general addition.
//            2b (k_window_running_sums): two warps per (row, window): lane k of the 64 takes the
//            magnitudes (64 k, 64 k + 64] from the top with the running-sum rule (run += bucket,
//            tot += run), adds 64 k * run, and each warp adds up its 32 totals;
//   stage 3  the finalize kernel of the fixed-base path recombines the windows (Horner) and adds
//            the shared point of the padded columns.
//
// Cost per row in mixed-addition times: about 1.2 * elements (stage 1) + n_bins * (1.3 + 20 * 1.27)
// instead of elements * windows.  The result is the same group element, so the normalised record is
// bit-identical.
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

// Stage 1 sums.  One thread: BS_ENTRIES consecutive table entries of one row, walked as one flat
// list of elements; Px[row][t] = sum of the generators of the row's elements with index t (XYZZ,
// infinity when the entry does not occur).
constexpr int BS_ENTRIES = 32;
__global__ void __launch_bounds__(128, 4) k_bucket_sums(const Affine* __restrict__ gens, const uint32_t* __restrict__ offs,
                                                     const uint32_t* __restrict__ sorted, uint32_t wd, uint32_t n_bins,
                                                     uint64_t n_threads, Xyzz* __restrict__ Px) {
  const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= n_threads) return;
  const uint32_t per_row = n_bins / BS_ENTRIES;
  const uint64_t row = gid / per_row;
  const uint32_t t0 = (uint32_t)(gid % per_row) * BS_ENTRIES, t1 = t0 + BS_ENTRIES;
  const uint32_t* orow = offs + row * (uint64_t)(n_bins + 1);
  const uint32_t* srow = sorted + row * wd;
  Xyzz* prow = Px + row * n_bins;
  uint32_t t = t0;
  uint32_t pos = orow[t0];
  uint32_t next = orow[t0 + 1];  // one past the last element of entry t
  Xyzz acc = Xyzz::inf();
  for (;;) {
    while (pos == next) {  // entry t is complete (possibly empty)
      xyzz_canon(acc).store(prow + t);   // the walk keeps lazy residues
      acc = Xyzz::inf();
      t++;
      if (t == t1) return;
      next = orow[t + 1];
    }
    xyzz_madd_lazy(acc, Affine::load_nc(gens + srow[pos]));
    pos++;
  }
}

// Px (XYZZ) -> P (affine, (0,0) for infinity), NORM_BATCH consecutive points per inversion.
constexpr int NORM_BATCH = 16;
__global__ void __launch_bounds__(128) k_normalise(const Xyzz* __restrict__ Px, uint64_t n, Affine* __restrict__ P) {
  const uint64_t i0 = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * NORM_BATCH;
  if (i0 >= n) return;
  const int cnt = (int)min((uint64_t)NORM_BATCH, n - i0);
  Fp pref[NORM_BATCH];
  Fp run = Fp::one();
#pragma unroll 1
  for (int k = 0; k < cnt; k++) {
    const char* e = reinterpret_cast<const char*>(Px + i0 + k);
    const Fp zzz = Fp::load(e + 2 * Fp::BYTES), zz = Fp::load(e + 3 * Fp::BYTES);
    if (!zz.is_zero()) run = fe_mul(run, fe_mul(zz, zzz));
    pref[k] = run;
  }
  Fp inv = fe_inv(run);
#pragma unroll 1
  for (int k = cnt - 1; k >= 0; k--) {
    const Xyzz e = Xyzz::load(Px + i0 + k);
    Affine out = Affine::inf();
    if (!e.is_inf()) {
      const Fp zinv = (k == 0) ? inv : fe_mul(inv, pref[k - 1]);  // 1 / (zz * zzz) of point k
      inv = fe_mul(inv, fe_mul(e.zz, e.zzz));
      out.x = fe_mul(e.x, fe_mul(zinv, e.zzz));
      out.y = fe_mul(e.y, fe_mul(zinv, e.zz));
    }
    out.store(P + i0 + k);
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

// ent[w][pos] = (table entry | sign << 31, magnitude) of the pos-th entry of window w in ascending
// order of magnitude: what a lane of stage 2a needs for one step, in one 8-byte load.
__global__ void k_pack_entries(const uint32_t* __restrict__ sorted2, const uint32_t* __restrict__ mags,
                               const uint8_t* __restrict__ neg, uint32_t n_bins, uint2* __restrict__ ent) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (uint64_t)STAGE2_WINDOWS * n_bins) return;
  const uint64_t w = i / n_bins;
  const uint32_t t = sorted2[i];
  ent[i] = make_uint2(t | ((uint32_t)neg[w * n_bins + t] << 31), mags[w * n_bins + t]);
}

// Stage 2a.  One lane: slice k of window w of one row.  The slice covers whole magnitudes: it starts
// after the first magnitude at which the running count of the window's entries reaches k * L and ends
// at the first at which it reaches (k + 1) * L, so every magnitude belongs to exactly one lane and a
// slice is within one bucket length of L entries.  S[row][w][m - 1] = sum of the +-P_t of magnitude m;
// magnitudes that no entry has keep the zeros (= infinity) the buffer was cleared to.
constexpr int WB_THREADS = 128;
__global__ void __launch_bounds__(WB_THREADS, 4)
k_window_buckets(const Affine* __restrict__ P, uint32_t n_bins, const uint32_t* __restrict__ offs2,
                 const uint2* __restrict__ ent, uint32_t slices, uint32_t slice_len, uint64_t n_threads,
                 Xyzz* __restrict__ S) {
  const uint64_t gid = (uint64_t)blockIdx.x * WB_THREADS + threadIdx.x;
  if (gid >= n_threads) return;
  const uint32_t k = (uint32_t)(gid % slices);
  const uint64_t rw = gid / slices;
  const uint32_t w = (uint32_t)(rw % STAGE2_WINDOWS);
  const uint64_t row = rw / STAGE2_WINDOWS;
  const uint32_t* o2 = offs2 + (uint64_t)w * (STAGE2_HALF + 2);
  const uint32_t first = __ldg(o2 + 1);                  // entries with a zero digit come first
  const uint32_t cnt = __ldg(o2 + STAGE2_HALF + 1) - first;
  // smallest magnitude m in [0, HALF] with (number of entries of magnitude 1..m) >= target
  auto bound = [&](uint64_t target) -> uint32_t {
    if (target >= cnt) target = cnt;
    uint32_t lo = 0, hi = STAGE2_HALF;
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if ((uint64_t)(__ldg(o2 + mid + 1) - first) >= target) hi = mid;
      else lo = mid + 1;
    }
    return lo;
  };
  const uint32_t m_lo = bound((uint64_t)k * slice_len);
  const uint32_t m_hi = (k + 1 == slices) ? STAGE2_HALF : bound((uint64_t)(k + 1) * slice_len);
  uint32_t pos = __ldg(o2 + m_lo + 1);
  const uint32_t end = __ldg(o2 + m_hi + 1);
  if (pos >= end) return;
  const uint2* e = ent + (uint64_t)w * n_bins;
  const Affine* prow = P + row * n_bins;
  Xyzz* srow = S + (row * STAGE2_WINDOWS + w) * STAGE2_HALF;
  uint32_t m_cur = 0;
  Xyzz run = Xyzz::inf();
  for (; pos < end; pos++) {
    const uint2 en = __ldg(e + pos);
    if (en.y != m_cur) {
      if (m_cur) xyzz_canon(run).store(srow + (m_cur - 1));
      run = Xyzz::inf();
      m_cur = en.y;
    }
    Affine p = Affine::load_nc(prow + (en.x & 0x7fffffffu));
    if (en.x >> 31) p.y = fe_neg(p.y);  // the point at infinity is (0, 0) and stays so
    xyzz_madd_lazy(run, p);
  }
  xyzz_canon(run).store(srow + (m_cur - 1));
}

// Stage 2b.  RS_SPLIT warps per (row, window): sum over magnitudes m of m * S_m.  Lane k of the
// RS_SPLIT * 32 lanes of a (row, window) takes the magnitudes (base, base + RS_PER_LANE], base =
// RS_PER_LANE * k, from the top with the running-sum rule, which leaves tot = sum (m - base) * S_m and
// run = sum S_m; base * run is added by double-and-add over the bits of k followed by log2(RS_PER_LANE)
// doublings; a shuffle tree adds the 32 totals of a warp and the warps of a (row, window) leave one
// partial sum each for the finalize kernel.  Two warps of 64 magnitudes per lane instead of one of 128:
// twice as many units, half as long, so the partial last wave of the grid costs half as much.
constexpr int RS_THREADS = 128;
constexpr uint32_t RS_SPLIT = 2;
constexpr uint32_t RS_PER_LANE = STAGE2_HALF / (32 * RS_SPLIT);
__global__ void __launch_bounds__(RS_THREADS, 3)
k_window_running_sums(const Xyzz* __restrict__ S, uint64_t n_units, Xyzz* __restrict__ partial) {
  const uint64_t unit = (uint64_t)blockIdx.x * (RS_THREADS / 32) + (threadIdx.x >> 5);  // (row, window, part)
  if (unit >= n_units) return;  // whole warps leave together
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t part = (uint32_t)(unit % RS_SPLIT);
  const uint32_t k = part * 32 + lane;  // index of this lane's magnitude range inside the window
  const Xyzz* s = S + (unit / RS_SPLIT) * STAGE2_HALF + (uint64_t)k * RS_PER_LANE;
  Xyzz run = Xyzz::inf(), tot = Xyzz::inf();
#pragma unroll 1
  for (int m = (int)RS_PER_LANE - 1; m >= 0; m--) {
    xyzz_add(run, Xyzz::load(s + m));
    xyzz_add(tot, run);
  }
  if (k != 0 && !run.is_inf()) {
    Xyzz acc = Xyzz::inf();
#pragma unroll 1
    for (int bit = 31 - __clz(k); bit >= 0; bit--) {
      acc = xyzz_dbl(acc);
      if ((k >> bit) & 1u) xyzz_add(acc, run);
    }
#pragma unroll 1
    for (uint32_t v = RS_PER_LANE; v > 1; v >>= 1) acc = xyzz_dbl(acc);
    xyzz_add(tot, acc);
  }
#pragma unroll 1
  for (int off = 16; off > 0; off >>= 1) {
    Xyzz other = xyzz_shfl_down(tot, off);
    if (lane < (uint32_t)off) xyzz_add(tot, other);
  }
  if (lane == 0) tot.store(partial + unit);
}

// Row commitments  C_row = sum_i B[idx[row][i]] * G_i  (+ extra, the same point for every row).
//   d_idx: [size] table indices, 0xFFFFFFFF for elements that take no part; d_B: n_bins Fr scalars.
// Returns GRAPE_ERR_INVALID when the shape is not supported (the caller then commits directly).
int commit_gathered_async(grape_ctx* ctx, const grape_table* t, const uint32_t* d_idx, const uint32_t* d_B,
                          uint32_t n_bins, uint64_t size, uint32_t wd, const void* d_extra, void* d_out) {
  static_assert(STAGE2_HALF % (32 * RS_SPLIT) == 0 && (RS_PER_LANE & (RS_PER_LANE - 1)) == 0, "stage 2b lane ranges");
  if (!t || t->curve != Bn254::ID || wd == 0 || wd > t->n_gens || size % wd != 0 || n_bins < BS_ENTRIES ||
      n_bins % BS_ENTRIES != 0 || n_bins > (1u << 24))
    return GRAPE_ERR_INVALID;
  const uint64_t rows = size / wd;
  if (rows == 0) return GRAPE_OK;
  if (rows > 0x7fffffffull) return GRAPE_ERR_INVALID;
  int rc;
  uint32_t *offs, *sorted, *mags, *offs2, *sorted2;
  uint8_t* neg;
  uint2* ent;
  Affine* P;
  Xyzz *Px, *S, *partial;
  // rows per pass of stage 2: bounds the bucket-sum buffer (10.5 MB per row) to about 1.3 GB
  const uint64_t batch = std::min<uint64_t>(rows, 128);
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)(n_bins + 1), &offs))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)wd, &sorted))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)n_bins, &P))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * (uint64_t)n_bins, &Px))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &mags))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &neg))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * (STAGE2_HALF + 2), &offs2))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &sorted2))) return rc;
  if ((rc = arena_alloc_t(ctx, (uint64_t)STAGE2_WINDOWS * n_bins, &ent))) return rc;
  if ((rc = arena_alloc_t(ctx, batch * STAGE2_WINDOWS * STAGE2_HALF, &S))) return rc;
  if ((rc = arena_alloc_t(ctx, rows * STAGE2_WINDOWS * RS_SPLIT, &partial))) return rc;
  GRAPE_CUDA_TRY(ctx, cudaFuncSetAttribute(k_row_sort, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(SORT_PART_BINS * sizeof(uint32_t))));
  // stage 1
  {
    const uint32_t parts = (n_bins + SORT_PART_BINS - 1) / SORT_PART_BINS;
    const size_t smem = (size_t)std::min(n_bins, SORT_PART_BINS) * sizeof(uint32_t);
    k_row_sort<<<dim3((uint32_t)rows, parts), SORT_THREADS, smem, ctx->stream>>>(d_idx, wd, n_bins, offs, sorted);
    const Affine* gens = reinterpret_cast<const Affine*>(t->data) + (uint64_t)t->first_digit_row * t->n_gens;
    const uint64_t n_threads = rows * (n_bins / BS_ENTRIES);
    k_bucket_sums<<<(uint32_t)((n_threads + 127) / 128), 128, 0, ctx->stream>>>(gens, offs, sorted, wd, n_bins,
                                                                                 n_threads, Px);
    const uint64_t n_pts = rows * (uint64_t)n_bins;
    const uint64_t norm_threads = (n_pts + NORM_BATCH - 1) / NORM_BATCH;
    k_normalise<<<(uint32_t)((norm_threads + 127) / 128), 128, 0, ctx->stream>>>(Px, n_pts, P);
    ctx->launches += 3;
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
    const uint64_t n_ent = (uint64_t)STAGE2_WINDOWS * n_bins;
    k_pack_entries<<<(uint32_t)((n_ent + 255) / 256), 256, 0, ctx->stream>>>(sorted2, mags, neg, n_bins, ent);
    ctx->launches += 3;
    // slices of about 256 entries: long enough that a lane's last partial step and the spread of slice
    // lengths inside a warp stay small, short enough that one row fills 20 * n_bins / 256 lanes
    const uint32_t slice_len = 256;
    const uint32_t slices = (n_bins + slice_len - 1) / slice_len;
    for (uint64_t r0 = 0; r0 < rows; r0 += batch) {
      const uint64_t nr = std::min<uint64_t>(batch, rows - r0);
      GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(S, 0, nr * STAGE2_WINDOWS * STAGE2_HALF * sizeof(Xyzz), ctx->stream));
      const uint64_t n_threads = nr * STAGE2_WINDOWS * slices;
      {
        ProfScope prof(ctx);
        k_window_buckets<<<(uint32_t)((n_threads + WB_THREADS - 1) / WB_THREADS), WB_THREADS, 0, ctx->stream>>>(
            P + r0 * n_bins, n_bins, offs2, ent, slices, slice_len, n_threads, S);
      }
      const uint64_t n_units = nr * STAGE2_WINDOWS * RS_SPLIT;
      k_window_running_sums<<<(uint32_t)((n_units + RS_THREADS / 32 - 1) / (RS_THREADS / 32)), RS_THREADS, 0,
                              ctx->stream>>>(S, n_units, partial + r0 * STAGE2_WINDOWS * RS_SPLIT);
      ctx->launches += 2;
    }
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  // stage 3: Horner over the windows, extra point, normalisation
  return finalize_bn254_async(ctx, partial, RS_SPLIT, STAGE2_WINDOWS, STAGE2_BITS, rows, d_out, d_extra);
}

}  // namespace grape
