// Hyrax row commitments: fixed-base multi-scalar multiplication over G1 of BN254 (the curve the
// reference compiles) or BLS12-381 (same kernels instantiated on the 12-limb base field).
//
// Replaces (paths inside the reference project):
//   precompute_generators / naive_msm                 src/ec_operation.cu:15-49
//   Hyrax::commit(int*) + int_windows_sum/_reduce     src/Hyrax.cu:312-333, 46-87
//   Hyrax::commit(FrTensor&) + many_windows_sum/_reduce  src/Hyrax.cu:335-359, 128-167
//   single_commit + single_windows_sum/_reduce        src/Hyrax.cu:176-185, 89-126
//
// Design.  All rows of a Hyrax commitment share the same generators, so the generators are
// expanded once into a table of small multiples and every (scalar, generator) pair costs one
// table gather and one mixed addition per non-zero signed digit.  Signed digits halve the table;
// with 16-bit windows an int16-range scalar is a single digit, i.e. a single addition per pair,
// at the price of a table of 2^15 rows that lives in HBM rather than in L2.
//
//   commit_accumulate:  one WARP per (row, window group, chunk of generators), four warps per
//                       block; a window group is the set of windows the table stores pre-shifted
//                       (all of them for 16-bit windows over int16 data).  A lane walks its
//                       generators with stride 32 and keeps one XYZZ accumulator (lazy residues) -- it
//                       never doubles; the block's 128 lane sums are paired off through shared
//                       memory (six warp-wide general additions) and one thread per warp writes
//                       the partial sum to scratch memory.
//   commit_accumulate_affine (msm_affine.cuh, selectable): the same sums with affine accumulators
//                       kept in device memory and one inversion shared by a batch of rows.
//   commit_finalize:    one thread per row recombines the groups (Horner: window_bits * n_windows
//                       doublings between groups, paid once per row instead of once per lane),
//                       adds the chunk partials, normalises (one inversion) and writes the
//                       canonical Jacobian record.
#include <algorithm>
#include <mutex>

#include "ctx.cuh"
#include "curve.cuh"

namespace grape {

template <class F>
struct TableViewT {
  const AffineT<F>* base;
  uint32_t n_gens;
  uint32_t window_bits;    // c
  uint32_t n_windows;      // windows whose 2^(c*w) multiples are stored
  uint32_t half;           // 2^(c-1): largest digit magnitude
  uint64_t window_stride;  // records per window
  uint32_t first_row;      // row of magnitude 1
  __device__ __forceinline__ const AffineT<F>* entry(uint32_t w, uint32_t mag, uint32_t i) const {
    return base + (uint64_t)w * window_stride + (uint64_t)(mag - 1 + first_row) * n_gens + i;
  }
};

using TableView = TableViewT<Fp>;

template <class F>
static TableViewT<F> make_view(const grape_table* t) {
  TableViewT<F> v;
  v.base = reinterpret_cast<const AffineT<F>*>(t->data);
  v.n_gens = t->n_gens;
  v.window_bits = t->window_bits;
  v.n_windows = t->n_windows;
  v.half = 1u << (t->window_bits - 1);
  v.window_stride = t->window_stride;
  v.first_row = t->first_digit_row;
  return v;
}

// ------------------------------------------------------------------------------------------
// Table construction
// ------------------------------------------------------------------------------------------
constexpr int TABLE_BLOCK = 16;  // consecutive multiples produced (and batch-normalised) per thread

// One thread: generator i, window w, magnitudes d0+1 .. d0+TABLE_BLOCK.
template <class C>
__global__ void __launch_bounds__(128) table_build_kernel(const JacobianT<typename C::F>* __restrict__ gens,
                                                          AffineT<typename C::F>* __restrict__ table,
                                                          uint32_t n_gens, uint32_t window_bits,
                                                          uint32_t n_windows, uint32_t half) {
  using Fp = typename C::F;
  using Jacobian = JacobianT<Fp>;
  using Affine = AffineT<Fp>;
  using Xyzz = XyzzT<Fp>;
  const uint32_t blocks_per_window = half / TABLE_BLOCK;
  uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint64_t total = (uint64_t)n_gens * n_windows * blocks_per_window;
  if (gid >= total) return;
  uint32_t i = gid % n_gens;
  uint64_t rest = gid / n_gens;
  uint32_t blk = rest % blocks_per_window;
  uint32_t w = rest / blocks_per_window;

  Jacobian gj;
  const char* gp = reinterpret_cast<const char*>(gens + i);
  gj.x = Fp::load(gp);
  gj.y = Fp::load(gp + Fp::BYTES);
  gj.z = Fp::load(gp + 2 * Fp::BYTES);
  Xyzz b = xyzz_from_jacobian(gj);
  for (uint32_t k = 0; k < window_bits * w; k++) b = xyzz_dbl(b);
  Affine base = xyzz_to_affine(b);  // 2^(c w) * G_i

  // start = d0 * base by double-and-add
  uint32_t d0 = blk * TABLE_BLOCK;
  Xyzz acc = Xyzz::inf();
  for (int bit = 15; bit >= 0; bit--) {
    acc = xyzz_dbl(acc);
    if ((d0 >> bit) & 1u) xyzz_madd(acc, base);
  }

  Xyzz e[TABLE_BLOCK];
  Fp pref[TABLE_BLOCK];
  Fp run = Fp::one();
#pragma unroll 1
  for (int k = 0; k < TABLE_BLOCK; k++) {
    xyzz_madd(acc, base);
    e[k] = acc;
    Fp zp = acc.is_inf() ? Fp::one() : fe_mul(acc.zz, acc.zzz);
    run = fe_mul(run, zp);
    pref[k] = run;
  }
  Fp inv = fe_inv(run);
  uint64_t wbase = (uint64_t)w * half * n_gens;
#pragma unroll 1
  for (int k = TABLE_BLOCK - 1; k >= 0; k--) {
    Fp zp = e[k].is_inf() ? Fp::one() : fe_mul(e[k].zz, e[k].zzz);
    Fp zinv = (k == 0) ? inv : fe_mul(inv, pref[k - 1]);  // 1 / (zz*zzz) of entry k
    inv = fe_mul(inv, zp);
    Affine out;
    if (e[k].is_inf()) {
      out = Affine::inf();
    } else {
      out.x = fe_mul(e[k].x, fe_mul(zinv, e[k].zzz));
      out.y = fe_mul(e[k].y, fe_mul(zinv, e[k].zz));
    }
    out.store(table + wbase + (uint64_t)(d0 + k) * n_gens + i);
  }
}

// ------------------------------------------------------------------------------------------
// Scalar preparation for Fr scalars: leave Montgomery form, add the signed-digit bias and cut the
// value into its signed c-bit digits ONCE, stored window-major as 16-bit integers
// (digits[w][element]).  Window e_w = bits [c w, c w + c) of (v + bias) gives digit e_w - 2^(c-1)
// (the top window is read unsigned).  The accumulate kernel then reads one digit per addition with
// consecutive lanes on consecutive addresses, where reading the 32-byte scalar again for every window
// group cost two scattered 4-byte loads per addition.
// ------------------------------------------------------------------------------------------
struct Bias256 {
  uint32_t v[8];
};

template <class C>
__global__ void fr_digits_kernel(const uint32_t* __restrict__ in, int16_t* __restrict__ digits, uint64_t n,
                                 Bias256 bias, uint32_t c, uint32_t total_windows) {
  using Fr = typename C::S;
  uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= n) return;
  Fr s = Fr::load_nc(in + gid * 8);
  s = fe_from_mont(s);
  uint32_t r[8];
  add8(r, s.v, bias.v);  // value < 2^255 and bias < 2^255: no carry out
  const uint32_t mask = (1u << c) - 1u, half = 1u << (c - 1);
  for (uint32_t w = 0; w < total_windows; w++) {
    const uint32_t bit = c * w, word = bit >> 5;
    const uint32_t lo = word < 8 ? r[word] : 0u, hi = word < 7 ? r[word + 1] : 0u;
    const uint32_t e = __funnelshift_r(lo, hi, bit & 31) & mask;
    const int32_t d = (w + 1 == total_windows) ? (int32_t)e : (int32_t)e - (int32_t)half;
    digits[(uint64_t)w * n + gid] = (int16_t)d;
  }
}

// 2^(c-1) at the bottom of every window below the top one
static Bias256 make_bias(uint32_t c, uint32_t total_windows) {
  Bias256 b;
  for (int k = 0; k < 8; k++) b.v[k] = 0;
  for (uint32_t w = 0; w + 1 < total_windows; w++) {
    uint32_t bit = c * w + c - 1;
    b.v[bit >> 5] |= 1u << (bit & 31);
  }
  return b;
}

// ------------------------------------------------------------------------------------------
// Accumulation
// ------------------------------------------------------------------------------------------
constexpr int MSM_THREADS = 128;

// Signed digit of window w.  Int32 path: |s| carries the sign separately.
struct DigitI32 {
  uint32_t vb;     // |s| + bias
  bool neg;
  __device__ __forceinline__ void load(const int32_t* p, uint32_t bias) {
    int32_t s = __ldg(p);
    neg = s < 0;
    uint32_t v = neg ? (0u - (uint32_t)s) : (uint32_t)s;
    vb = v + bias;
  }
};

// Signed digit of window w of |s| + bias (int32 scalars; the sign of s is applied by the caller).
__device__ __forceinline__ int32_t i32_digit(uint32_t vb, uint32_t w, uint32_t c, uint32_t mask, uint32_t half,
                                             uint32_t total_windows) {
  const uint32_t sh = c * w;
  if (w + 1 == total_windows) return (int32_t)(sh < 32 ? (vb >> sh) : 0u);
  return (int32_t)((vb >> sh) & mask) - (int32_t)half;
}

}  // namespace grape
#include "msm_affine.cuh"
namespace grape {

// The 32 lane sums of each of the block's four warps become one partial sum per warp through shared
// memory: the 128 sums are paired off by as few threads as there are pairs (64, 32, 16, 8, 4), which
// costs the block six warp-wide general additions where a shuffle tree inside every warp costs twenty
// (measured on the 49 408 x 4096 workload: 34.2 ms against 35.8 ms).  Prefetching the next table record
// into L2 or L1 was measured too and lost 2 to 3 %: the gathers are already hidden by the other warps.
template <class C, bool FR>
__global__ void __launch_bounds__(MSM_THREADS, C::MSM_BLOCKS)
commit_accumulate_kernel(const void* __restrict__ scalars, TableViewT<typename C::F> tab, uint32_t wd,
                         uint32_t total_windows, uint32_t n_chunks, uint32_t chunk_len,
                         uint64_t n_units, XyzzT<typename C::F>* __restrict__ partials,
                         uint32_t* __restrict__ status, uint32_t inner, uint32_t inner_pad, uint64_t n_scalars) {
  using Affine = AffineT<typename C::F>;
  using Xyzz = XyzzT<typename C::F>;
  const uint64_t unit0 = (uint64_t)blockIdx.x * (MSM_THREADS / 32);
  const uint64_t unit = unit0 + (threadIdx.x >> 5);
  const bool live = unit < n_units;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t c = tab.window_bits;
  const uint32_t mask = (1u << c) - 1u;
  const uint32_t half = tab.half;
  const uint32_t tw = tab.n_windows;
  const uint32_t groups = (total_windows + tw - 1) / tw;
  // unit = (row, window group, chunk of generators): no doubling happens here; the finalize kernel
  // recombines the groups of a row with c * tw doublings between them
  const uint32_t chunk = (uint32_t)(unit % n_chunks);
  const uint64_t rg = unit / n_chunks;
  const uint32_t g = (uint32_t)(rg % groups);
  const uint64_t row = rg / groups;
  // With inner != 0 (Fr scalars only) a row is sub-rows of inner_pad columns of which only the first
  // `inner` are walked: the caller accounts for the skipped (constant) columns separately.
  const uint32_t wd_walk = (FR && inner) ? wd / inner_pad * inner : wd;
  const uint32_t i_begin = chunk * chunk_len;
  const uint32_t i_end = live ? min(wd_walk, i_begin + chunk_len) : 0u;

  // bias for the int32 path: 2^(c-1) at every window below the top one
  uint32_t bias32 = 0;
  if (!FR) {
    for (uint32_t w = 0; w + 1 < total_windows; w++) bias32 |= half << (c * w);
  }
  const uint32_t w_lo = g * tw;
  const uint32_t w_hi = min(total_windows, w_lo + tw);
  auto column = [&](uint32_t j) -> uint32_t {
    if (FR && inner) {
      const uint32_t q = j / inner;
      return q * inner_pad + (j - q * inner);
    }
    return j;
  };

  Xyzz acc = Xyzz::inf();
  for (uint32_t j = i_begin + lane; j < i_end; j += 32) {
    const uint32_t i = column(j);
    const uint64_t idx = row * wd + i;
    if (FR) {
      // scalars = the digit planes written by fr_digits_kernel: digits[w][element], n_scalars elements each
      const int16_t* dp = reinterpret_cast<const int16_t*>(scalars) + idx;
      for (uint32_t w = w_lo; w < w_hi; w++) {
        const int32_t d = __ldg(dp + (uint64_t)w * n_scalars);
        if (d == 0) continue;
        uint32_t mag = d < 0 ? (uint32_t)(-d) : (uint32_t)d;
        Affine p = Affine::load_nc(tab.entry(w - w_lo, mag, i));
        if (d < 0) p.y = fe_neg(p.y);
        xyzz_madd_lazy(acc, p);
      }
    } else {
      DigitI32 dg;
      dg.load(reinterpret_cast<const int32_t*>(scalars) + idx, bias32);
      for (uint32_t w = w_lo; w < w_hi; w++) {
        const int32_t d = i32_digit(dg.vb, w, c, mask, half, total_windows);
        if (d == 0) continue;
        uint32_t mag = d < 0 ? (uint32_t)(-d) : (uint32_t)d;
        if (mag > half) {  // scalar larger than the declared bound: report, never read out of range
          atomicOr(status, STATUS_DIGIT_RANGE);
          continue;
        }
        Affine p = Affine::load_nc(tab.entry(w - w_lo, mag, i));
        if ((d < 0) != dg.neg) p.y = fe_neg(p.y);
        xyzz_madd_lazy(acc, p);
      }
    }
  }

  {
    // The pool holds the 128 lane sums as 16-byte pieces, piece k of slot t at pool4[k * 128 + t]:
    // consecutive lanes touch consecutive 16-byte words (a record-per-thread layout would put all lanes
    // of a quarter warp on the same four banks).
    constexpr int PIECES = sizeof(Xyzz) / 16;
    __shared__ uint4 pool4[PIECES * MSM_THREADS];
    auto put = [&](uint32_t slot, const Xyzz& p) {
      const uint4* src = reinterpret_cast<const uint4*>(&p);
#pragma unroll
      for (int k = 0; k < PIECES; k++) pool4[k * MSM_THREADS + slot] = src[k];
    };
    auto get = [&](uint32_t slot) {
      Xyzz p;
      uint4* dst = reinterpret_cast<uint4*>(&p);
#pragma unroll
      for (int k = 0; k < PIECES; k++) dst[k] = pool4[k * MSM_THREADS + slot];
      return p;
    };
    const uint32_t tid = threadIdx.x;
    put(tid, xyzz_canon(acc));   // the loop keeps lazy residues; everything downstream is canonical
    __syncthreads();
#pragma unroll 1
    for (uint32_t width = 16; width >= 1; width >>= 1) {
      if (tid < (MSM_THREADS / 32) * width) {
        const uint32_t u = tid / width, k = tid - u * width;
        Xyzz a = get(u * 32 + k);
        xyzz_add(a, get(u * 32 + k + width));
        if (width == 1) {
          if (unit0 + u < n_units) a.store(partials + unit0 + u);
        } else {
          put(u * 32 + k, a);
        }
      }
      __syncthreads();
    }
  }
}

// One thread per row: result = sum over window groups g of 2^(group_bits * g) * (sum of the row's
// chunk partials of group g), evaluated top group first with group_bits doublings in between.
// partials are laid out [row][group][chunk].
template <class C>
__global__ void __launch_bounds__(128) commit_finalize_kernel(const XyzzT<typename C::F>* __restrict__ partials,
                                                              uint32_t n_chunks, uint32_t groups,
                                                              uint32_t group_bits, uint64_t rows,
                                                              JacobianT<typename C::F>* __restrict__ out,
                                                              const JacobianT<typename C::F>* __restrict__ extra) {
  using Affine = AffineT<typename C::F>;
  using Xyzz = XyzzT<typename C::F>;
  uint64_t row = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  Xyzz acc = Xyzz::inf();
  // one serial stream per thread: the field operations are calls so that the loop stays in the
  // instruction cache
#pragma unroll 1
  for (int g = (int)groups - 1; g >= 0; g--) {
    if (g != (int)groups - 1) {
#pragma unroll 1
      for (uint32_t k = 0; k < group_bits; k++) acc = xyzz_dbl_compact(acc);
    }
    const Xyzz* p = partials + (row * groups + (uint32_t)g) * n_chunks;
#pragma unroll 1
    for (uint32_t k = 0; k < n_chunks; k++) xyzz_add_compact(acc, Xyzz::load(p + k));
  }
  if (extra) {  // the same point added to every row (the constant columns skipped by the accumulation)
    JacobianT<typename C::F> e;
    const char* ep = reinterpret_cast<const char*>(extra);
    e.x = C::F::load(ep);
    e.y = C::F::load(ep + C::F::BYTES);
    e.z = C::F::load(ep + 2 * C::F::BYTES);
    xyzz_add(acc, xyzz_from_jacobian(e));
  }
  bool inf = acc.is_inf();
  Affine a = xyzz_to_affine(acc);
  store_jacobian_normalised(out + row, a, inf);
}

// The same for commitments of FEW rows (openings commit a single row split into hundreds of chunks):
// one block per row.  Warp k adds the chunk partials of groups k, k + 8, ... with a strided loop and a
// shuffle tree, leaves each group sum in shared memory, and thread 0 runs the Horner recombination.
constexpr int FIN_THREADS = 256;
constexpr int FIN_MAX_GROUPS = 64;

template <class C>
__global__ void __launch_bounds__(FIN_THREADS) commit_finalize_block_kernel(
    const XyzzT<typename C::F>* __restrict__ partials, uint32_t n_chunks, uint32_t groups, uint32_t group_bits,
    JacobianT<typename C::F>* __restrict__ out, const JacobianT<typename C::F>* __restrict__ extra) {
  using Affine = AffineT<typename C::F>;
  using Xyzz = XyzzT<typename C::F>;
  __shared__ __align__(16) unsigned char sums_raw[FIN_MAX_GROUPS * sizeof(Xyzz)];
  Xyzz* sums = reinterpret_cast<Xyzz*>(sums_raw);
  const uint64_t row = blockIdx.x;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t g = warp; g < groups; g += FIN_THREADS / 32) {
    const Xyzz* p = partials + (row * groups + g) * n_chunks;
    Xyzz acc = Xyzz::inf();
#pragma unroll 1
    for (uint32_t k = lane; k < n_chunks; k += 32) xyzz_add(acc, Xyzz::load(p + k));
#pragma unroll 1
    for (int off = 16; off > 0; off >>= 1) {
      Xyzz other = xyzz_shfl_down(acc, off);
      if (lane < off) xyzz_add(acc, other);
    }
    if (lane == 0) acc.store(sums + g);
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  Xyzz acc = Xyzz::inf();
#pragma unroll 1
  for (int g = (int)groups - 1; g >= 0; g--) {
    if (g != (int)groups - 1) {
#pragma unroll 1
      for (uint32_t k = 0; k < group_bits; k++) acc = xyzz_dbl_compact(acc);
    }
    xyzz_add_compact(acc, Xyzz::load(sums + g));
  }
  if (extra) {
    JacobianT<typename C::F> e;
    const char* ep = reinterpret_cast<const char*>(extra);
    e.x = C::F::load(ep);
    e.y = C::F::load(ep + C::F::BYTES);
    e.z = C::F::load(ep + 2 * C::F::BYTES);
    xyzz_add(acc, xyzz_from_jacobian(e));
  }
  bool inf = acc.is_inf();
  Affine a = xyzz_to_affine(acc);
  store_jacobian_normalised(out + row, a, inf);
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
static int check_table(grape_ctx* ctx, const grape_table* t, uint32_t wd) {
  if (!ctx || !t || !t->data) return fail(ctx, GRAPE_ERR_INVALID, "null context or table");
  if (wd == 0 || wd > t->n_gens)
    return fail(ctx, GRAPE_ERR_INVALID, "row length exceeds the number of generators in the table");
  return GRAPE_OK;
}

// Picks how many warps (chunks of generators) share one (row, window group).
//   * Few units (less than half of the warps the GPU holds at once): enough chunks to reach that, while
//     every lane keeps at least two generators.  More lose: every chunk pays its share of the block
//     reduction (measured on 1024 rows of 1024 generators: one chunk 0.29 ms, five chunks 0.42 ms).
//   * Fewer than two waves of units: cut them until there are two, as long as a chunk keeps 2048
//     generators (64 additions per lane, the reduction stays near 3 % of a unit).
//   * Otherwise one chunk.  Cutting units further to shorten the partial last wave of a grid was
//     measured and does not pay: with 24 704 rows of 4096 generators two chunks per row took 16.9 ms
//     where one chunk took half of the 49 408-row launch plus 1.4 % (the end of a grid is already
//     staggered, and every chunk adds its reduction).
static uint32_t pick_chunks(const grape_ctx* ctx, uint64_t rows, uint32_t wd, uint32_t groups = 1) {
  const uint64_t cap = (uint64_t)ctx->sm_count * 16;  // resident warps: four blocks of four per SM
  const uint64_t units = rows * groups;               // every (row, window group) is a unit of its own
  if (units == 0) return 1;
  uint64_t want = 1, max_chunks = 1;
  if (units < cap / 2) {
    want = (cap / 2 + units - 1) / units;
    max_chunks = (wd + 63) / 64;
  } else if (units < 2 * cap) {
    want = (2 * cap + units - 1) / units;
    max_chunks = wd / 2048;
  }
  if (want > max_chunks) want = max_chunks;
  if (want < 1) want = 1;
  return (uint32_t)want;
}

template <class C, bool FR>
static int launch_commit(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t rows,
                         uint32_t wd, uint32_t total_windows, XyzzT<typename C::F>* partials,
                         uint32_t n_chunks, void* d_out, uint32_t inner = 0, uint32_t inner_pad = 0,
                         const void* d_extra = nullptr, const AffinePlan* plan = nullptr, uint4* aff_scratch = nullptr) {
  const uint32_t wd_walk = inner ? wd / inner_pad * inner : wd;
  uint32_t chunk_len = (wd_walk + n_chunks - 1) / n_chunks;
  const uint32_t groups = (total_windows + t->n_windows - 1) / t->n_windows;
  uint64_t units = rows * groups * n_chunks;
  if (units == 0) return GRAPE_OK;
  uint64_t blocks = (units + MSM_THREADS / 32 - 1) / (MSM_THREADS / 32);
  if (blocks > 0x7fffffffull) return fail(ctx, GRAPE_ERR_LIMIT, "too many commitment rows for one launch");
  if (plan && plan->use) {
    AffineArgs<typename C::F> a;
    a.scalars = d_scalars;
    a.tab = make_view<typename C::F>(t);
    a.wd = wd;
    a.total_windows = total_windows;
    a.groups = groups;
    a.n_chunks = plan->n_chunks;
    a.chunk_len = plan->chunk_len;
    a.n_slots = rows * groups;
    a.n_units = plan->units;
    a.B = plan->B;
    a.partials = partials;
    a.status = ctx->d_status;
    a.inner = inner;
    a.inner_pad = inner_pad;
    a.n_scalars = rows * (uint64_t)wd;
    a.scratch = aff_scratch;
    const uint32_t grid = (uint32_t)((plan->grid_warps + AFF_THREADS / 32 - 1) / (AFF_THREADS / 32));
    ProfScope prof(ctx);
    commit_accumulate_affine_kernel<C, FR><<<grid, AFF_THREADS, 0, ctx->stream>>>(a);
  } else {
    ProfScope prof(ctx);
    commit_accumulate_kernel<C, FR><<<(uint32_t)blocks, MSM_THREADS, 0, ctx->stream>>>(
        d_scalars, make_view<typename C::F>(t), wd, total_windows, n_chunks, chunk_len, units, partials,
        ctx->d_status, inner, inner_pad, rows * (uint64_t)wd);
  }
  const JacobianT<typename C::F>* extra = reinterpret_cast<const JacobianT<typename C::F>*>(d_extra);
  if (n_chunks >= 8 && groups <= FIN_MAX_GROUPS && rows <= 4096)
    commit_finalize_block_kernel<C><<<(uint32_t)rows, FIN_THREADS, 0, ctx->stream>>>(
        partials, n_chunks, groups, t->window_bits * t->n_windows, reinterpret_cast<JacobianT<typename C::F>*>(d_out),
        extra);
  else
    commit_finalize_kernel<C><<<(uint32_t)((rows + 127) / 128), 128, 0, ctx->stream>>>(
        partials, n_chunks, groups, t->window_bits * t->n_windows, rows,
        reinterpret_cast<JacobianT<typename C::F>*>(d_out), extra);
  ctx->launches += 2;
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

// Chooses between the two accumulation kernels for `rows` rows and carves the scratch either needs.
template <class C>
static int plan_commit(grape_ctx* ctx, const grape_table* t, uint64_t rows, uint32_t wd_walk, uint32_t groups,
                       bool fr_scalars, AffinePlan* plan, uint32_t* n_chunks, XyzzT<typename C::F>** partials,
                       uint4** aff_scratch) {
  *plan = AffinePlan();
  *aff_scratch = nullptr;
  const int mode = fr_scalars ? ctx->affine_mode_fr : ctx->affine_mode;
  // below a few million additions the extended-coordinate kernel fills the GPU better
  if (mode == 2 || (mode == 1 && (uint64_t)rows * groups * wd_walk * t->n_windows >= (1ull << 22)))
    *plan = plan_affine(ctx, rows * groups, wd_walk, t->n_windows, mode == 2, mode == 2 ? ctx->affine_b : 0,
                        mode == 2 ? ctx->affine_chunks : 0);
  *n_chunks = plan->use ? plan->n_chunks : pick_chunks(ctx, rows, wd_walk, groups);
  int rc = arena_alloc_t(ctx, rows * groups * *n_chunks, partials);
  if (rc) return rc;
  if (plan->use) {
    constexpr size_t rec = 3 * (C::F::BYTES / 16) * 32 * sizeof(uint4);
    void* p = nullptr;
    if ((rc = arena_alloc(ctx, (size_t)plan->grid_warps * plan->B * rec, &p))) return rc;
    *aff_scratch = reinterpret_cast<uint4*>(p);
  }
  return GRAPE_OK;
}

}  // namespace grape

namespace grape {

template <class C>
static int table_create_impl(grape_ctx* ctx, const void* d_gens_jacobian, uint32_t n_gens, uint32_t window_bits,
                             uint32_t n_windows, grape_table** out) {
  using AffineC = AffineT<typename C::F>;
  using JacobianC = JacobianT<typename C::F>;
  if (!ctx || !out || !d_gens_jacobian) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (window_bits < 5 || window_bits > 16)
    return fail(ctx, GRAPE_ERR_INVALID, "window_bits must be between 5 and 16");
  if (n_gens == 0 || n_windows == 0 || n_windows * window_bits > 256)
    return fail(ctx, GRAPE_ERR_INVALID, "bad table geometry");
  uint32_t half = 1u << (window_bits - 1);
  uint64_t records = (uint64_t)half * n_gens * n_windows;
  void* data = nullptr;
  cudaError_t e = cudaMalloc(&data, records * sizeof(AffineC));
  if (e != cudaSuccess) return fail(ctx, GRAPE_ERR_NOMEM, "generator table allocation failed");
  uint64_t threads = (uint64_t)n_gens * n_windows * (half / TABLE_BLOCK);
  uint64_t blocks = (threads + 127) / 128;
  if (blocks > 0x7fffffffull) {
    cudaFree(data);
    return fail(ctx, GRAPE_ERR_LIMIT, "table too large for one launch");
  }
  table_build_kernel<C><<<(uint32_t)blocks, 128, 0, ctx->stream>>>(
      reinterpret_cast<const JacobianC*>(d_gens_jacobian), reinterpret_cast<AffineC*>(data), n_gens,
      window_bits, n_windows, half);
  ctx->launches += 1;
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) {
    cudaFree(data);
    return fail(ctx, GRAPE_ERR_CUDA, std::string("table_build_kernel: ") + cudaGetErrorString(le));
  }
  grape_table* t = new grape_table();
  t->ctx = ctx;
  t->data = data;
  t->owned = true;
  t->n_gens = n_gens;
  t->window_bits = window_bits;
  t->n_windows = n_windows;
  t->n_digits = half;
  t->window_stride = (uint64_t)half * n_gens;
  t->first_digit_row = 0;
  t->curve = C::ID;
  *out = t;
  return GRAPE_OK;
}

template <class C>
static int commit_i32_impl(grape_ctx* ctx, const grape_table* t, const int32_t* d_scalars, uint64_t rows,
                           uint32_t wd, uint32_t max_bits, void* d_out) {
  uint32_t total_windows = (max_bits + t->window_bits - 1) / t->window_bits;
  const uint32_t groups = (total_windows + t->n_windows - 1) / t->n_windows;
  arena_reset(ctx);
  AffinePlan plan;
  uint32_t n_chunks = 1;
  XyzzT<typename C::F>* partials = nullptr;
  uint4* aff = nullptr;
  int rc = plan_commit<C>(ctx, t, rows, wd, groups, false, &plan, &n_chunks, &partials, &aff);
  if (rc) return rc;
  return launch_commit<C, false>(ctx, t, d_scalars, rows, wd, total_windows, partials, n_chunks, d_out, 0, 0, nullptr,
                                 &plan, aff);
}

// The number of windows is chosen so that window_bits * windows exceeds the scalar width: the top
// window is read unsigned and then never exceeds the largest stored magnitude.
template <class C>
static int commit_fr_impl(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size,
                          uint64_t rows, uint32_t wd, void* d_out, uint32_t inner = 0, uint32_t inner_pad = 0,
                          const void* d_extra = nullptr) {
  uint32_t total_windows = (C::SCALAR_BITS + t->window_bits) / t->window_bits;
  if (C::ID == Bn254::ID) total_windows = (254 + t->window_bits - 1) / t->window_bits;
  const uint32_t groups = (total_windows + t->n_windows - 1) / t->n_windows;
  const uint32_t wd_walk = inner ? wd / inner_pad * inner : wd;
  AffinePlan plan;
  uint32_t n_chunks = 1;
  XyzzT<typename C::F>* partials = nullptr;
  uint4* aff = nullptr;
  int16_t* digits = nullptr;
  int rc = plan_commit<C>(ctx, t, rows, wd_walk, groups, true, &plan, &n_chunks, &partials, &aff);
  if (rc) return rc;
  rc = arena_alloc_t(ctx, size * total_windows, &digits);
  if (rc) return rc;
  fr_digits_kernel<C><<<(uint32_t)((size + 255) / 256), 256, 0, ctx->stream>>>(
      reinterpret_cast<const uint32_t*>(d_scalars), digits, size, make_bias(t->window_bits, total_windows),
      t->window_bits, total_windows);
  ctx->launches += 1;
  return launch_commit<C, true>(ctx, t, digits, rows, wd, total_windows, partials, n_chunks, d_out, inner, inner_pad,
                               d_extra, &plan, aff);
}

static size_t jacobian_bytes(const grape_table* t) {
  return t->curve == Bls12381::ID ? sizeof(JacobianT<BlsFp>) : sizeof(Jacobian);
}

}  // namespace grape

using namespace grape;

extern "C" int grape_table_create(grape_ctx* ctx, const void* d_gens_jacobian, uint32_t n_gens,
                                  uint32_t window_bits, uint32_t n_windows, grape_table** out) {
  if (ctx) grape::make_device_current(ctx);
  return table_create_impl<Bn254>(ctx, d_gens_jacobian, n_gens, window_bits, n_windows, out);
}

extern "C" int grape_bls12_381_table_create(grape_ctx* ctx, const void* d_gens_jacobian, uint32_t n_gens,
                                            uint32_t window_bits, uint32_t n_windows, grape_table** out) {
  if (ctx) grape::make_device_current(ctx);
  return table_create_impl<Bls12381>(ctx, d_gens_jacobian, n_gens, window_bits, n_windows, out);
}

extern "C" int grape_table_from_reference(grape_ctx* ctx, const void* d_points, uint32_t n_gens,
                                          grape_table** out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !out || !d_points || n_gens == 0) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  grape_table* t = new grape_table();
  t->ctx = ctx;
  t->data = const_cast<void*>(d_points);
  t->owned = false;
  t->n_gens = n_gens;
  t->window_bits = 8;
  t->n_windows = 1;
  t->n_digits = 128;
  t->window_stride = (uint64_t)256 * n_gens;
  t->first_digit_row = 1;  // row 0 of that layout is 0*G = infinity
  t->curve = Bn254::ID;
  *out = t;
  return GRAPE_OK;
}

extern "C" int grape_table_destroy(grape_table* t) {
  if (!t) return GRAPE_OK;
  if (t->owned && t->data) cudaFree(t->data);
  delete t;
  return GRAPE_OK;
}

extern "C" uint64_t grape_table_bytes(const grape_table* t) {
  if (!t) return 0;
  uint64_t rows = t->owned ? (uint64_t)t->n_digits * t->n_windows : 256;
  return rows * t->n_gens * (t->curve == Bls12381::ID ? sizeof(AffineT<BlsFp>) : sizeof(Affine));
}

extern "C" const void* grape_table_data(const grape_table* t) { return t ? t->data : nullptr; }

extern "C" uint32_t grape_table_curve(const grape_table* t) { return t ? t->curve : 0; }

extern "C" int grape_commit_i32(grape_ctx* ctx, const grape_table* t, const int32_t* d_scalars,
                                uint64_t size, uint32_t wd, uint32_t max_bits, void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  int rc = check_table(ctx, t, wd);
  if (rc) return rc;
  if (size % wd != 0) return fail(ctx, GRAPE_ERR_INVALID, "size is not a multiple of the row length");
  if (max_bits == 0 || max_bits > 32) return fail(ctx, GRAPE_ERR_INVALID, "max_bits must be in 1..32");
  if (size == 0) return GRAPE_OK;
  if (!d_scalars || !d_out) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  uint64_t rows = size / wd;
  if (t->curve == Bls12381::ID) return commit_i32_impl<Bls12381>(ctx, t, d_scalars, rows, wd, max_bits, d_out);
  return commit_i32_impl<Bn254>(ctx, t, d_scalars, rows, wd, max_bits, d_out);
}

namespace grape {
// Fr-scalar commitment that takes its scratch from the arena without resetting it (used inside the
// lookup prover, which holds other arena regions at that point).
int commit_fr_async(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size, uint32_t wd,
                    void* d_out) {
  int rc = check_table(ctx, t, wd);
  if (rc) return rc;
  if (size % wd != 0) return fail(ctx, GRAPE_ERR_INVALID, "size is not a multiple of the row length");
  if (size == 0) return GRAPE_OK;
  if (!d_scalars || !d_out) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  uint64_t rows = size / wd;
  if (t->curve == Bls12381::ID) return commit_fr_impl<Bls12381>(ctx, t, d_scalars, size, rows, wd, d_out);
  return commit_fr_impl<Bn254>(ctx, t, d_scalars, size, rows, wd, d_out);
}
}  // namespace grape

namespace grape {

// ones[i] = 1 on the constant columns (i mod inner_pad >= inner), 0 elsewhere
__global__ void k_constant_columns(int32_t* __restrict__ ones, uint32_t wd, uint32_t inner, uint32_t inner_pad) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < wd; i += gridDim.x * blockDim.x)
    ones[i] = (i % inner_pad) >= inner ? 1 : 0;
}

// out = [s] * P (Jacobian record in, normalised Jacobian record out), one thread: 254 doublings.
__global__ void k_scale_point(const uint32_t* __restrict__ point_jac, const uint32_t* __restrict__ scalar,
                              uint32_t* __restrict__ out_jac) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  Jacobian j;
  j.x = Fp::load(point_jac);
  j.y = Fp::load(point_jac + 8);
  j.z = Fp::load(point_jac + 16);
  Xyzz base = xyzz_from_jacobian(j);
  Fr s = fe_from_mont(Fr::load(scalar));
  Xyzz acc = Xyzz::inf();
#pragma unroll 1
  for (int w = 7; w >= 0; w--) {
#pragma unroll 1
    for (int b = 31; b >= 0; b--) {
      acc = xyzz_dbl_compact(acc);
      if ((s.v[w] >> b) & 1u) xyzz_add_compact(acc, base);
    }
  }
  bool inf = acc.is_inf();
  Affine a = xyzz_to_affine(acc);
  store_jacobian_normalised(out_jac, a, inf);
}

// The point  s_const * (sum of the generators of the constant columns)  of rows that are sub-rows of
// inner_pad columns whose columns past `inner` all hold the scalar at d_const: a one-row commitment
// of 0/1 scalars and one scalar multiplication.  *d_point: a Jacobian record in the arena.
int constant_columns_point_async(grape_ctx* ctx, const grape_table* t, uint32_t wd, uint32_t inner, uint32_t inner_pad,
                                 const void* d_const, uint32_t** d_point) {
  int rc;
  int32_t* ones = nullptr;
  uint32_t* pts = nullptr;  // sum of the constant columns' generators | that sum times the constant
  if ((rc = arena_alloc_t(ctx, (size_t)wd, &ones))) return rc;
  if ((rc = arena_alloc_t(ctx, 2 * 24 + 8, &pts))) return rc;
  k_constant_columns<<<std::min<uint32_t>((wd + 255) / 256, 1024u), 256, 0, ctx->stream>>>(ones, wd, inner, inner_pad);
  ctx->launches += 1;
  const uint32_t n_chunks = pick_chunks(ctx, 1, wd, 1);
  Xyzz* partials = nullptr;
  if ((rc = arena_alloc_t(ctx, (size_t)n_chunks, &partials))) return rc;
  if ((rc = launch_commit<Bn254, false>(ctx, t, ones, 1, wd, 1, partials, n_chunks, pts))) return rc;
  k_scale_point<<<1, 32, 0, ctx->stream>>>(pts, reinterpret_cast<const uint32_t*>(d_const), pts + 24);
  ctx->launches += 1;
  *d_point = pts + 24;
  return GRAPE_OK;
}

// Row commitments of a tensor whose rows are sub-rows of inner_pad columns where every column past
// `inner` holds the SAME scalar (the row padding of the lookup arguments: about a third of a
// 11008 -> 16384 padded row).  The constant columns contribute one point for all rows, added by
// the finalize kernel, while the accumulation walks the first `inner` columns of each sub-row only.
int commit_fr_padded_async(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size, uint32_t wd,
                           uint32_t inner, uint32_t inner_pad, const void* d_const, void* d_out) {
  if (inner == 0 || inner >= inner_pad || wd % inner_pad != 0 || t->curve != Bn254::ID)
    return commit_fr_async(ctx, t, d_scalars, size, wd, d_out);
  int rc = check_table(ctx, t, wd);
  if (rc) return rc;
  if (size % wd != 0) return fail(ctx, GRAPE_ERR_INVALID, "size is not a multiple of the row length");
  if (size == 0) return GRAPE_OK;
  uint32_t* point = nullptr;
  if ((rc = constant_columns_point_async(ctx, t, wd, inner, inner_pad, d_const, &point))) return rc;
  return commit_fr_impl<Bn254>(ctx, t, d_scalars, size, size / wd, wd, d_out, inner, inner_pad, point);
}

// Horner recombination + normalisation of partial sums laid out [row][group][chunk] (BN254).
int finalize_bn254_async(grape_ctx* ctx, const Xyzz* partials, uint32_t n_chunks, uint32_t groups, uint32_t group_bits,
                         uint64_t rows, void* d_out, const void* d_extra) {
  if (rows == 0) return GRAPE_OK;
  const Jacobian* extra = reinterpret_cast<const Jacobian*>(d_extra);
  if (n_chunks >= 8 && groups <= FIN_MAX_GROUPS && rows <= 4096)
    commit_finalize_block_kernel<Bn254><<<(uint32_t)rows, FIN_THREADS, 0, ctx->stream>>>(
        partials, n_chunks, groups, group_bits, reinterpret_cast<Jacobian*>(d_out), extra);
  else
    commit_finalize_kernel<Bn254><<<(uint32_t)((rows + 127) / 128), 128, 0, ctx->stream>>>(
        partials, n_chunks, groups, group_bits, rows, reinterpret_cast<Jacobian*>(d_out), extra);
  ctx->launches += 1;
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

}  // namespace grape

extern "C" int grape_commit_fr(grape_ctx* ctx, const grape_table* t, const void* d_scalars,
                               uint64_t size, uint32_t wd, void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx) return GRAPE_ERR_INVALID;
  arena_reset(ctx);
  return commit_fr_async(ctx, t, d_scalars, size, wd, d_out);
}

extern "C" int grape_commit_i32_host(grape_ctx* ctx, const grape_table* t, const int32_t* h_scalars,
                                     uint64_t size, uint32_t wd, uint32_t max_bits, void* h_out) {
  if (ctx) grape::make_device_current(ctx);
  int rc = check_table(ctx, t, wd);
  if (rc) return rc;
  if (size % wd != 0) return fail(ctx, GRAPE_ERR_INVALID, "size is not a multiple of the row length");
  if (size == 0) return GRAPE_OK;
  uint64_t rows = size / wd;
  size_t in_bytes = size * sizeof(int32_t);
  const size_t jac = jacobian_bytes(t);
  size_t out_bytes = rows * jac;
  // Page-locked scalars are read by the kernel where they lie: every scalar is needed exactly once, the
  // other warps of an SM cover the longer latency of a read across PCIe, and no slice waits for a copy
  // (measured on 49 408 rows: 33.3 ms against 34.7 ms for the sliced copies below and 32.3 ms with the
  // scalars already in device memory).  Pageable buffers take the staged path.
  {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, h_scalars) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr) {
      if (out_bytes > ctx->dstage_bytes) {
        GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->dstage) cudaFree(ctx->dstage);
        ctx->dstage = nullptr;
        ctx->dstage_bytes = 0;
        if (cudaMalloc(&ctx->dstage, out_bytes) != cudaSuccess)
          return fail(ctx, GRAPE_ERR_NOMEM, "staging buffer allocation failed");
        ctx->dstage_bytes = out_bytes;
      }
      rc = grape_commit_i32(ctx, t, reinterpret_cast<const int32_t*>(attr.devicePointer), size, wd, max_bits,
                            ctx->dstage);
      if (rc) return rc;
      GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_out, ctx->dstage, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
      GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
      return GRAPE_OK;
    }
    cudaGetLastError();  // a pointer the runtime does not know is not an error here
  }
  size_t need = ((in_bytes + 255) & ~size_t(255)) + out_bytes;
  if (need > ctx->dstage_bytes) {
    GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->dstage) cudaFree(ctx->dstage);
    ctx->dstage = nullptr;
    ctx->dstage_bytes = 0;
    if (cudaMalloc(&ctx->dstage, need) != cudaSuccess)
      return fail(ctx, GRAPE_ERR_NOMEM, "staging buffer allocation failed");
    ctx->dstage_bytes = need;
  }
  int32_t* d_in = reinterpret_cast<int32_t*>(ctx->dstage);
  char* d_out = reinterpret_cast<char*>(ctx->dstage) + ((in_bytes + 255) & ~size_t(255));
  // Row slices: slice i+1 is copied in on the copy stream while slice i is being committed.  The
  // copy runs about 2.4x faster than the commitment, so only the first slice's copy is exposed: it is
  // kept small (1/32 of the rows) and the later slices grow, which keeps their launches long enough
  // to fill whole waves of warps.
  static const uint32_t kSliceParts[5] = {1, 3, 7, 10, 11};  // of 32
  const uint32_t n_slices = rows >= 4096 ? 5 : 1;
  if (!ctx->copy_stream) GRAPE_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  while (ctx->copy_events.size() < n_slices + 1) {
    cudaEvent_t e;
    GRAPE_CUDA_TRY(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    ctx->copy_events.push_back(e);
  }
  uint64_t bounds[6];
  bounds[0] = 0;
  for (uint32_t sidx = 0, acc = 0; sidx < n_slices; sidx++) {
    acc += kSliceParts[sidx];
    bounds[sidx + 1] = n_slices == 1 ? rows : rows * acc / 32;
  }
  bounds[n_slices] = rows;
  // the copy stream must not overwrite the staging buffer while earlier work still reads it
  GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[n_slices], ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_events[n_slices], 0));
  for (uint32_t sidx = 0; sidx < n_slices; sidx++) {
    const uint64_t r0 = bounds[sidx], r1 = bounds[sidx + 1];
    if (r1 > r0)
      GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_in + r0 * wd, h_scalars + r0 * wd, (r1 - r0) * wd * sizeof(int32_t),
                                          cudaMemcpyHostToDevice, ctx->copy_stream));
    GRAPE_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_events[sidx], ctx->copy_stream));
  }
  for (uint32_t sidx = 0; sidx < n_slices; sidx++) {
    const uint64_t r0 = bounds[sidx], r1 = bounds[sidx + 1];
    GRAPE_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->copy_events[sidx], 0));
    if (r1 == r0) continue;
    rc = grape_commit_i32(ctx, t, d_in + r0 * wd, (r1 - r0) * wd, wd, max_bits, d_out + r0 * jac);
    if (rc) return rc;
  }
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_out, d_out, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return GRAPE_OK;
}

// ------------------------------------------------------------------------------------------
// Commitment without any allocation
// ------------------------------------------------------------------------------------------
// For callers that must not allocate device memory at the moment they commit: code that runs
// inside a memory-pool-managed framework where a stray cudaMalloc would synchronise the device
// or fragment the pool, latency-critical serving loops, and hosts whose GPU memory is already
// fully handed out to other buffers.  The per-(row, chunk) partial sums that the other entry
// points keep in the context's scratch arena live here in a fixed array inside the library image.
// Every GPU that loads the library holds that array (GRAPE_STATIC_SCRATCH_BYTES) until exit.
constexpr uint64_t STATIC_MAX_UNITS = 65536;  // rows x window groups x chunks per call
static __device__ __align__(256) unsigned char g_static_partials[STATIC_MAX_UNITS * sizeof(grape::Xyzz)];
static __device__ __align__(256) uint32_t g_static_status[64];

namespace {
struct StaticDeviceState {
  bool ready = false;
  void* partials = nullptr;  // device address of g_static_partials on this device
  uint32_t* status = nullptr;
  int sm_count = 0;
};
StaticDeviceState g_static_state[64];
std::mutex g_static_mutex;                  // guards the once-per-device set-up below
thread_local char g_static_error[256] = "";  // text of the calling thread's last failure

// Resolves the device addresses of the static arrays for the CURRENT device, once per device.
// In host code the array names are only stand-ins; the kernels must be given these addresses.
int static_setup(int device, StaticDeviceState** out) {
  if (device < 0 || device >= 64) {
    snprintf(g_static_error, sizeof g_static_error, "device index %d out of range", device);
    return GRAPE_ERR_LIMIT;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticDeviceState& st = g_static_state[device];
  if (!st.ready) {
    void* p = nullptr;
    void* s = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_partials);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&s, g_static_status);
    int sms = 0;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) {
      snprintf(g_static_error, sizeof g_static_error, "static scratch set-up failed: %s", cudaGetErrorString(e));
      return GRAPE_ERR_CUDA;
    }
    st.partials = p;
    st.status = reinterpret_cast<uint32_t*>(s);
    st.sm_count = sms;
    st.ready = true;
  }
  *out = &st;
  return GRAPE_OK;
}
}  // namespace

extern "C" uint64_t grape_static_scratch_bytes(void) { return sizeof(g_static_partials); }
extern "C" const char* grape_static_error(void) { return g_static_error; }

// Same result as grape_commit_i32, for a BN254 table laid out as grape_table_create builds it
// (d_table = grape_table_data, same n_gens / window_bits / n_windows; NOT a BLS12-381 table and NOT
// the 256-row layout grape_table_from_reference wraps: the raw pointer carries neither fact, so a
// wrong table is read as garbage), on the current device and the given stream (NULL = default stream).  It calls no cudaMalloc, cudaFree or any routine
// that allocates; inputs, outputs and the table are the caller's.
//   * Limit: rows * window groups * chunks <= 65536 partial sums (rows = size / wd, window groups =
//     ceil(ceil(max_bits / window_bits) / n_windows), chunks = what fills the GPU when there are
//     few rows); rows * window groups > 65536 is rejected with GRAPE_ERR_LIMIT (text in
//     grape_static_error()).
//   * The first call on a device resolves the address of the library's static scratch for that
//     device (cudaGetSymbolAddress with that device current); make that first call outside any
//     stream capture.
//   * All calls on a device share the one static array, which keeps whatever the previous call
//     left in it.  Each call overwrites every partial it later reads and clears the status word
//     first, so back-to-back calls on one stream are fine; two calls whose kernels can overlap
//     on the GPU (different streams, different threads) race on it.
//   * h_status (may be NULL): if given, the call synchronises the stream and stores 1 there when
//     some scalar exceeded max_bits (that scalar's out-of-range digit is skipped), else 0.  Without
//     it an out-of-range scalar goes unreported: the flag lives in the static status word, which the
//     next call clears.
//   * Host threads: the per-device set-up is serialised and grape_static_error() is per thread, so
//     the entry point may be called from several threads; their kernels still share the one array.
extern "C" int grape_commit_i32_static(const void* d_table, uint32_t n_gens, uint32_t window_bits,
                                       uint32_t n_windows, const int32_t* d_scalars, uint64_t size, uint32_t wd,
                                       uint32_t max_bits, void* d_out, void* stream, uint32_t* h_status) {
  if (!d_table || !d_scalars || !d_out) {
    snprintf(g_static_error, sizeof g_static_error, "null argument");
    return GRAPE_ERR_INVALID;
  }
  if (window_bits < 5 || window_bits > 16 || n_windows == 0 || n_windows * window_bits > 256 || wd == 0 ||
      wd > n_gens || size % wd != 0 || max_bits == 0 || max_bits > 32) {
    snprintf(g_static_error, sizeof g_static_error, "bad geometry (window_bits 5..16, n_windows * window_bits <= 256, wd <= n_gens, size %% wd == 0, max_bits 1..32)");
    return GRAPE_ERR_INVALID;
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    snprintf(g_static_error, sizeof g_static_error, "no current CUDA device");
    return GRAPE_ERR_CUDA;
  }
  StaticDeviceState* st = nullptr;
  int rc = static_setup(device, &st);
  if (rc) return rc;
  const uint64_t rows = size / wd;
  if (rows == 0) return GRAPE_OK;
  // chunks per (row, window group): as in the arena-backed path, but capped by the static array
  const uint32_t total_windows = (max_bits + window_bits - 1) / window_bits;
  const uint32_t groups = (total_windows + n_windows - 1) / n_windows;
  const uint64_t row_units = rows * groups;
  uint64_t target_warps = (uint64_t)st->sm_count * 8;
  uint64_t n_chunks = 1;
  if (row_units < target_warps) {
    n_chunks = std::min<uint64_t>((target_warps + row_units - 1) / row_units, (wd + 63) / 64);
    if (n_chunks < 1) n_chunks = 1;
  }
  while (n_chunks > 1 && row_units * n_chunks > STATIC_MAX_UNITS) n_chunks--;
  if (row_units * n_chunks > STATIC_MAX_UNITS) {
    snprintf(g_static_error, sizeof g_static_error, "%llu rows x %u window group(s) exceed the static scratch limit of %llu partial sums",
             (unsigned long long)rows, groups, (unsigned long long)STATIC_MAX_UNITS);
    return GRAPE_ERR_LIMIT;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  TableView view;
  view.base = reinterpret_cast<const Affine*>(d_table);
  view.n_gens = n_gens;
  view.window_bits = window_bits;
  view.n_windows = n_windows;
  view.half = 1u << (window_bits - 1);
  view.window_stride = (uint64_t)view.half * n_gens;
  view.first_row = 0;
  const uint32_t chunk_len = (uint32_t)((wd + n_chunks - 1) / n_chunks);
  const uint64_t units = row_units * n_chunks;
  const uint64_t blocks = (units + MSM_THREADS / 32 - 1) / (MSM_THREADS / 32);
  Xyzz* partials = reinterpret_cast<Xyzz*>(st->partials);
  cudaError_t e = cudaMemsetAsync(st->status, 0, sizeof(uint32_t), s);  // must start at zero
  if (e == cudaSuccess) {
    commit_accumulate_kernel<Bn254, false><<<(uint32_t)blocks, MSM_THREADS, 0, s>>>(
        d_scalars, view, wd, total_windows, (uint32_t)n_chunks, chunk_len, units, partials, st->status, 0u, 0u,
        (uint64_t)0);
    commit_finalize_kernel<Bn254><<<(uint32_t)((rows + 127) / 128), 128, 0, s>>>(partials, (uint32_t)n_chunks, groups,
                                                                          window_bits * n_windows, rows,
                                                                          reinterpret_cast<Jacobian*>(d_out), nullptr);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess && h_status) {
    uint32_t flag = 0;
    e = cudaMemcpyAsync(&flag, st->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    *h_status = flag ? 1u : 0u;
  }
  if (e != cudaSuccess) {
    snprintf(g_static_error, sizeof g_static_error, "grape_commit_i32_static: %s", cudaGetErrorString(e));
    return GRAPE_ERR_CUDA;
  }
  return GRAPE_OK;
}
