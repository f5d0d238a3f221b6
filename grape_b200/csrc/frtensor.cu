// Field-tensor kernels over BN254 Fr (device arrays of 32-byte Montgomery residues).
//
// Replaces the FrTensor runtime of the reference (src/fr-tensor.cu): int -> Fr conversion
// (:30-46), Montgomery in/out (:110-120), element-wise and broadcast arithmetic (:74-108),
// inversion (:122-126), padding (:18-28), tree sum (:128-153, 415-440), row sums (:155-163) and
// the multilinear fold (:53-72, 168-188, 330-344).
//
// Differences in mechanism, not in results: kernels are grid-stride and sized to the SM count,
// loads/stores are 16-byte vectors, inversion is batched (Montgomery's trick across a block, one
// field inversion per 2048 elements), and the fold of an axis is a single pass that multiplies
// by a table of eq-weights instead of log2(c) in-place passes.
#include "ctx.cuh"
#include <algorithm>
#include "field.cuh"

namespace grape {

constexpr int EW_THREADS = 256;

static inline uint32_t ew_blocks(const grape_ctx* ctx, uint64_t n) {
  uint64_t b = (n + EW_THREADS - 1) / EW_THREADS;
  uint64_t cap = (uint64_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  if (b == 0) b = 1;
  return (uint32_t)b;
}

#define GRID_STRIDE(i, n) \
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (uint64_t)gridDim.x * blockDim.x)

__global__ void k_from_i32(const int32_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t n) {
  GRID_STRIDE(i, n) fe_from_i32<FrParams>(__ldg(in + i)).store(out + i * 8);
}
__global__ void k_from_u32(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t n) {
  GRID_STRIDE(i, n) fe_from_u32<FrParams>(__ldg(in + i)).store(out + i * 8);
}
__global__ void k_to_mont(uint32_t* t, uint64_t n) {
  GRID_STRIDE(i, n) fe_to_mont(Fr::load(t + i * 8)).store(t + i * 8);
}
__global__ void k_from_mont(uint32_t* t, uint64_t n) {
  GRID_STRIDE(i, n) fe_from_mont(Fr::load(t + i * 8)).store(t + i * 8);
}

template <int OP, class F>
__global__ void k_binary(const uint32_t* a, const uint32_t* b, uint32_t* out, uint64_t n) {
  GRID_STRIDE(i, n) {
    F x = F::load(a + i * 8), y = F::load(b + i * 8);
    F r = OP == 0 ? fe_add(x, y) : OP == 1 ? fe_sub(x, y) : fe_mul(x, y);
    r.store(out + i * 8);
  }
}

// out = a (op) s[0], s a device scalar
template <int OP>
__global__ void k_broadcast(const uint32_t* a, const uint32_t* __restrict__ s, uint32_t* out, uint64_t n) {
  Fr y = Fr::load_nc(s);
  GRID_STRIDE(i, n) {
    Fr x = Fr::load(a + i * 8);
    Fr r = OP == 0 ? fe_add(x, y) : fe_mul(x, y);
    r.store(out + i * 8);
  }
}

// out = a * s[0] + b     (z = c*x + d of the opening, src/Hyrax.cu:281-284)
__global__ void k_axpy(const uint32_t* a, const uint32_t* __restrict__ s, const uint32_t* b,
                       uint32_t* out, uint64_t n) {
  Fr y = Fr::load_nc(s);
  GRID_STRIDE(i, n) fe_add(fe_mul(Fr::load(a + i * 8), y), Fr::load(b + i * 8)).store(out + i * 8);
}

// Row padding: out[g] = (g % pad_n < n) ? in[(g / pad_n) * n + g % pad_n] : pad
__global__ void k_pad_i32(const int32_t* __restrict__ in, int32_t* __restrict__ out, uint32_t n,
                          uint32_t pad_n, uint64_t size) {
  GRID_STRIDE(g, size) {
    uint64_t r = g / pad_n, c = g % pad_n;
    out[g] = c < n ? __ldg(in + r * n + c) : 0;
  }
}
__global__ void k_pad_fr(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint32_t n,
                         uint32_t pad_n, uint64_t size, const uint32_t* __restrict__ pad) {
  Fr pv = Fr::load_nc(pad);
  GRID_STRIDE(g, size) {
    uint64_t r = g / pad_n, c = g % pad_n;
    Fr v = c < n ? Fr::load_nc(in + (r * n + c) * 8) : pv;
    v.store(out + g * 8);
  }
}

// ---- batched inversion --------------------------------------------------------------------
// out[i] = 1 / (in[i] + shift[0]); an element whose shifted value is zero maps to zero.
// Montgomery's trick per thread: thread t owns elements t, t+G, t+2G, ... (G = threads in the
// grid, so every access is coalesced), writes the running product before each element to scratch,
// inverts its total once, and unwinds in reverse.  About 3 multiplications per element plus one
// inversion per thread; `in` and `out` may be the same buffer.
__global__ void __launch_bounds__(128)
k_batch_inverse(const uint32_t* in, const uint32_t* __restrict__ shift, uint32_t* out,
                uint32_t* __restrict__ prefix, uint64_t n) {
  const uint64_t G = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const Fr sh = shift ? Fr::load_nc(shift) : Fr::zero();
  Fr run = Fr::one();
  uint64_t i = t;
  for (; i < n; i += G) {
    Fr v = fe_add(Fr::load(in + i * 8), sh);
    run.store(prefix + i * 8);
    if (!v.is_zero()) run = fe_mul(run, v);
  }
  Fr inv = fe_inv(run);
  // i is now the first index past the end for this thread; walk back
  while (i >= G + t) {
    i -= G;
    Fr v = fe_add(Fr::load(in + i * 8), sh);
    if (v.is_zero()) {
      Fr::zero().store(out + i * 8);
    } else {
      fe_mul(inv, Fr::load(prefix + i * 8)).store(out + i * 8);
      inv = fe_mul(inv, v);
    }
  }
}

// ---- sums -----------------------------------------------------------------------------------
constexpr int SUM_THREADS = 256;

__device__ __forceinline__ Fr block_sum(Fr acc) {
  __shared__ Fr warp_part[SUM_THREADS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc = fe_add(acc, fe_shfl_down(acc, off));
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    Fr v = threadIdx.x < (blockDim.x >> 5) ? warp_part[threadIdx.x] : Fr::zero();
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fe_add(v, fe_shfl_down(v, off));
    acc = v;
  }
  __syncthreads();
  return acc;  // valid in thread 0
}

__global__ void __launch_bounds__(SUM_THREADS) k_sum_partial(const uint32_t* __restrict__ in, uint64_t n,
                                                             uint32_t* __restrict__ partial) {
  Fr acc = Fr::zero();
  GRID_STRIDE(i, n) acc = fe_add(acc, Fr::load_nc(in + i * 8));
  acc = block_sum(acc);
  if (threadIdx.x == 0) acc.store(partial + (uint64_t)blockIdx.x * 8);
}

// Row sums broadcast back over the row (softmax denominator; reference sum_by_dim_kernel,
// src/fr-tensor.cu:155-163).  One warp per row.
__global__ void k_rowsum_broadcast(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                   uint64_t rows, uint32_t dim) {
  uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint32_t lane = threadIdx.x & 31;
  uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    Fr acc = Fr::zero();
    for (uint32_t i = lane; i < dim; i += 32) acc = fe_add(acc, Fr::load_nc(in + (r * dim + i) * 8));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc = fe_add(acc, fe_shfl_xor(acc, off));
    for (uint32_t i = lane; i < dim; i += 32) acc.store(out + (r * dim + i) * 8);
  }
}

// ---- sums of (field element) x (32-bit integer) without a reduction per term ------------------
// For folds that read int32 tensors.  acc += w * |x| with w a reduced residue (8 limbs) and |x| < 2^32:
// the 288-bit products are added into two interleaved accumulators (even limbs of w at limb
// offsets 0,2,4,6; odd limbs one limb higher), each with a 32-bit overflow word, so up to 2^32
// terms fit.  One term costs eight 32x32->64 multiply-adds; the value is reduced once at the end.
struct WideAcc {
  uint32_t E[8], O[8], Et, Ot;
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < 8; i++) { E[i] = 0; O[i] = 0; }
    Et = 0;
    Ot = 0;
  }
  __device__ __forceinline__ void mac(const Fr& w, uint32_t ax) {
    mad4_top(E, Et, w.v[0], w.v[2], w.v[4], w.v[6], ax);
    mad4_top(O, Ot, w.v[1], w.v[3], w.v[5], w.v[7], ax);
  }
  // The accumulated integer V = E + (O << 32) (320 bits) as the residue V mod r.  Because the
  // weights are Montgomery residues and the integers are plain, V mod r IS the Montgomery form of
  // the weighted sum.  V = V_a + 2^224 * V_b with V_a < 2^224 < r and V_b < 2^96, and
  // 2^224 * V_b mod r is ONE Montgomery product of V_b with the constant 2^480 mod r.
  __device__ __forceinline__ Fr to_fr() const {
    uint32_t L[10];
    uint64_t carry = 0;
    L[0] = E[0];
#pragma unroll
    for (int k = 1; k < 8; k++) {
      uint64_t s = (uint64_t)E[k] + O[k - 1] + carry;
      L[k] = (uint32_t)s;
      carry = s >> 32;
    }
    uint64_t s8 = (uint64_t)Et + O[7] + carry;
    L[8] = (uint32_t)s8;
    L[9] = Ot + (uint32_t)(s8 >> 32);
    const uint32_t t480[8] = {0x8f8fc595u, 0x41a9cbe4u, 0x0a58dc0fu, 0x9f36d601u,
                              0x440ad260u, 0xa6132126u, 0x093f81ddu, 0x2ab23b99u};  // 2^480 mod r
    Fr T, va = Fr::zero(), vb = Fr::zero();
#pragma unroll
    for (int k = 0; k < 8; k++) T.v[k] = t480[k];
#pragma unroll
    for (int k = 0; k < 7; k++) va.v[k] = L[k];
    vb.v[0] = L[7];
    vb.v[1] = L[8];
    vb.v[2] = L[9];
    return fe_add(va, fe_mul(vb, T));
  }
};

// Signed integers enter the wide sums biased: x + 2^31 is a plain 32-bit unsigned number, and
//   sum_j w_j x_j = sum_j w_j (x_j + 2^31) - 2^31 * sum_j w_j,
// where the last sum does not depend on the tensor: it is formed once per slice of j by this kernel
// (corr[s] = 2^31 * sum of w over slice s, a field element) and subtracted from every output.
__global__ void __launch_bounds__(SUM_THREADS) k_bias_correction(const uint32_t* __restrict__ w, uint32_t c,
                                                                 uint32_t slice_len, uint32_t* __restrict__ corr) {
  const uint32_t j0 = blockIdx.x * slice_len, j1 = min(c, j0 + slice_len);
  Fr acc = Fr::zero();
  for (uint32_t j = j0 + threadIdx.x; j < j1; j += SUM_THREADS) acc = fe_add(acc, Fr::load_nc(w + (uint64_t)j * 8));
  acc = block_sum(acc);
  if (threadIdx.x == 0) {
    Fr two31 = Fr::zero();
    two31.v[0] = 0x80000000u;
    fe_mul(acc, fe_to_mont(two31)).store(corr + (uint64_t)blockIdx.x * 8);
  }
}

// ---- multilinear fold ---------------------------------------------------------------------
// eq-weights of an axis of length c under challenges x[0..nv):  w[j] = prod_k (bit_k(j) ? x_k : 1 - x_k)
__global__ void k_eq_weights(const uint32_t* __restrict__ x, uint32_t nv, uint32_t c,
                             uint32_t* __restrict__ w) {
  GRID_STRIDE(j, c) {
    Fr acc = Fr::one();
    for (uint32_t k = 0; k < nv; k++) {
      Fr xk = Fr::load_nc(x + (uint64_t)k * 8);
      Fr f = ((j >> k) & 1) ? xk : fe_sub(Fr::one(), xk);
      acc = fe_mul(acc, f);
    }
    acc.store(w + j * 8);
  }
}

// out[o][g] (+)= sum_{j in slice} w[j] * t[o][j][g].   grid.x tiles the outputs, grid.y splits j.
// With one j-slice the result goes straight to `out`, otherwise to partial[slice][o*gap+g].
constexpr int FOLD_THREADS = 128;
template <bool FROM_I32>
__global__ void __launch_bounds__(FOLD_THREADS)
k_fold_axis(const void* __restrict__ t, const uint32_t* __restrict__ w, uint32_t c, uint64_t gap,
            uint64_t n_out, uint32_t slice_len, uint32_t* __restrict__ dst, const uint32_t* __restrict__ corr) {
  const uint64_t og = (uint64_t)blockIdx.x * FOLD_THREADS + threadIdx.x;
  if (og >= n_out) return;
  const uint64_t o = og / gap, g = og % gap;
  const uint32_t j0 = blockIdx.y * slice_len;
  const uint32_t j1 = min(c, j0 + slice_len);
  Fr acc = Fr::zero();
  if (FROM_I32) {
    // int32 source: 4 bytes and eight multiply-adds per element (biased to unsigned, see k_bias_correction)
    const int32_t* tp = reinterpret_cast<const int32_t*>(t) + (o * c + j0) * gap + g;
    const uint32_t* wp = w + (uint64_t)j0 * 8;
    WideAcc wide;
    wide.clear();
    constexpr int U = 8;  // loads in flight per thread (16 was slower)
    uint32_t j = j0;
    for (; j + U <= j1; j += U) {
      uint32_t xs[U];
#pragma unroll
      for (int k = 0; k < U; k++) xs[k] = (uint32_t)__ldg(tp + (uint64_t)k * gap) ^ 0x80000000u;
#pragma unroll
      for (int k = 0; k < U; k++) wide.mac(Fr::load_nc(wp + k * 8), xs[k]);
      tp += (uint64_t)U * gap;
      wp += U * 8;
    }
    for (; j < j1; j++) {
      wide.mac(Fr::load_nc(wp), (uint32_t)__ldg(tp) ^ 0x80000000u);
      tp += gap;
      wp += 8;
    }
    acc = fe_sub(wide.to_fr(), Fr::load_nc(corr + (uint64_t)blockIdx.y * 8));
  } else {
    for (uint32_t j = j0; j < j1; j++) {
      const uint64_t idx = (o * c + j) * gap + g;
      Fr v = Fr::load_nc(reinterpret_cast<const uint32_t*>(t) + idx * 8);
      acc = fe_add(acc, fe_mul(v, Fr::load_nc(w + (uint64_t)j * 8)));
    }
  }
  acc.store(dst + ((uint64_t)blockIdx.y * n_out + og) * 8);
}

// ---- int32-source fold staged through shared memory -------------------------------------------
// One block folds a tile of ST_COLS adjacent output columns over a slice of rows.  Rows arrive in
// shared memory by bulk asynchronous copies (cp.async.bulk, one per row chunk, completion counted on
// an mbarrier per stage), ST_STAGES stages of ST_ROWS rows deep, issued by one thread: the copies of
// a block stay in flight while all of its threads multiply, independent of how the compiler
// schedules loads, and a row chunk is one contiguous request.  The eq-weights of the stage's rows
// ride along in the same stage.  Every lane owns CPT adjacent columns (one 16-, 8- or 4-byte read of
// shared memory per row) and CPT wide accumulators.
// Every wait on an mbarrier is bounded: a lane that gives up sets STATUS_PIPE_TIMEOUT in the status
// word and the block leaves after a bounded wait for the copies it still has in flight.
constexpr int ST_ROWS = 8;
constexpr int ST_STAGES = 4;
constexpr uint32_t ST_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// false when the barrier did not complete the phase within the spin limit
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < ST_SPIN_LIMIT; spin++) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// global -> shared bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) of this GPU's own memory
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int CPT>
struct StageLayout {
  static constexpr int COLS = CPT * FOLD_THREADS;
  static constexpr int ROW_BYTES = COLS * 4;
  static constexpr int DATA_BYTES = ST_ROWS * ROW_BYTES;
  static constexpr int W_BYTES = ST_ROWS * 32;
  static constexpr int STAGE_BYTES = DATA_BYTES + W_BYTES;
  static constexpr int SMEM_BYTES = ST_STAGES * STAGE_BYTES + ST_STAGES * 8;
};

template <int CPT>
__global__ void __launch_bounds__(FOLD_THREADS)
k_fold_axis_i32_staged(const int32_t* __restrict__ t, const uint32_t* __restrict__ w, uint32_t c, uint64_t gap,
                       uint64_t n_out, uint32_t slice_len, uint32_t* __restrict__ dst, const uint32_t* __restrict__ corr,
                       uint32_t* __restrict__ status) {
  using L = StageLayout<CPT>;
  extern __shared__ __align__(128) unsigned char st_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(st_smem + ST_STAGES * L::STAGE_BYTES);
  const uint32_t tid = threadIdx.x;
  const uint64_t tiles_per_o = gap / L::COLS;
  const uint64_t o = blockIdx.x / tiles_per_o;
  const uint64_t g0 = (blockIdx.x % tiles_per_o) * L::COLS;
  const uint32_t j0 = blockIdx.y * slice_len;
  const uint32_t j1 = min(c, j0 + slice_len);
  const uint32_t n_rows = j1 > j0 ? j1 - j0 : 0;
  const uint32_t n_iter = (n_rows + ST_ROWS - 1) / ST_ROWS;
  const int32_t* src0 = t + (o * c + j0) * gap + g0;  // row j0 of this tile
  const uint32_t* w0 = w + (uint64_t)j0 * 8;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < ST_STAGES; s++) mbar_init(full + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](uint32_t it) {  // thread 0: fill stage it % ST_STAGES with rows it*ST_ROWS ...
    const uint32_t s = it % ST_STAGES;
    const uint32_t r0 = it * ST_ROWS;
    const uint32_t rows = min((uint32_t)ST_ROWS, n_rows - r0);
    unsigned char* base = st_smem + s * L::STAGE_BYTES;
    mbar_expect_tx(full + s, rows * (L::ROW_BYTES + 32));
    for (uint32_t r = 0; r < rows; r++)
      bulk_g2s(base + r * L::ROW_BYTES, src0 + (uint64_t)(r0 + r) * gap, L::ROW_BYTES, full + s);
    bulk_g2s(base + L::DATA_BYTES, w0 + (uint64_t)r0 * 8, rows * 32, full + s);
  };
  uint32_t issued = 0;
  if (tid == 0) {
    for (; issued < n_iter && issued < ST_STAGES; issued++) issue(issued);
  }

  WideAcc acc[CPT];
#pragma unroll
  for (int q = 0; q < CPT; q++) acc[q].clear();
  bool ok = true;
  for (uint32_t it = 0; it < n_iter; it++) {
    const uint32_t s = it % ST_STAGES;
    // the block decides together: a lane that ran out of patience must not leave the others at the
    // barrier below
    if (!__syncthreads_and(mbar_wait_bounded(full + s, (it / ST_STAGES) & 1u))) {
      ok = false;
      break;
    }
    const unsigned char* base = st_smem + s * L::STAGE_BYTES;
    const uint32_t rows = min((uint32_t)ST_ROWS, n_rows - it * ST_ROWS);
#pragma unroll 2
    for (uint32_t r = 0; r < rows; r++) {
      const Fr wk = Fr::load(base + L::DATA_BYTES + r * 32);
      const uint32_t* xr = reinterpret_cast<const uint32_t*>(base + r * L::ROW_BYTES) + tid * CPT;
      if (CPT == 4) {
        const uint4 x = *reinterpret_cast<const uint4*>(xr);
        acc[0].mac(wk, x.x ^ 0x80000000u);
        acc[1 % CPT].mac(wk, x.y ^ 0x80000000u);
        acc[2 % CPT].mac(wk, x.z ^ 0x80000000u);
        acc[3 % CPT].mac(wk, x.w ^ 0x80000000u);
      } else if (CPT == 2) {
        const uint2 x = *reinterpret_cast<const uint2*>(xr);
        acc[0].mac(wk, x.x ^ 0x80000000u);
        acc[1 % CPT].mac(wk, x.y ^ 0x80000000u);
      } else {
        acc[0].mac(wk, xr[0] ^ 0x80000000u);
      }
    }
    __syncthreads();  // every lane is done with stage s before it is refilled
    if (tid == 0 && issued < n_iter) issue(issued++);
  }
  if (!ok) {
    // a copy never completed: report, give the copies still in flight a bounded time to land, leave
    if (tid == 0) {
      atomicOr(status, STATUS_PIPE_TIMEOUT);
      for (int s = 0; s < ST_STAGES; s++) {
        mbar_wait_bounded(full + s, 0);
        mbar_wait_bounded(full + s, 1);
      }
    }
    return;
  }
  const Fr cr = Fr::load_nc(corr + (uint64_t)blockIdx.y * 8);
  const uint64_t og = o * gap + g0 + (uint64_t)tid * CPT;
  uint32_t* d = dst + ((uint64_t)blockIdx.y * n_out + og) * 8;
#pragma unroll
  for (int q = 0; q < CPT; q++) fe_sub(acc[q].to_fr(), cr).store(d + q * 8);
}

// out[i] = sum_s partial[s][i]
__global__ void k_sum_slices(const uint32_t* __restrict__ partial, uint32_t n_slices, uint64_t n,
                             uint32_t* __restrict__ out) {
  GRID_STRIDE(i, n) {
    Fr acc = Fr::load_nc(partial + i * 8);
    for (uint32_t s = 1; s < n_slices; s++) acc = fe_add(acc, Fr::load_nc(partial + ((uint64_t)s * n + i) * 8));
    acc.store(out + i * 8);
  }
}

// Innermost-axis fold (gap == 1): out[o] = sum_j w[j] * t[o*c + j], one block per o.
template <bool FROM_I32>
__global__ void __launch_bounds__(SUM_THREADS)
k_fold_inner(const void* __restrict__ t, const uint32_t* __restrict__ w, uint32_t c,
             uint32_t* __restrict__ out, const uint32_t* __restrict__ corr) {
  const uint64_t o = blockIdx.x;
  Fr acc = Fr::zero();
  if (FROM_I32) {
    // biased integers; the correction 2^31 * sum_j w_j is the same for every row (corr[0])
    const int32_t* ti = reinterpret_cast<const int32_t*>(t) + o * c;
    WideAcc wide;
    wide.clear();
    constexpr int U = 4;
    for (uint32_t jb = threadIdx.x; jb < c; jb += U * SUM_THREADS) {
      uint32_t xs[U];
#pragma unroll
      for (int k = 0; k < U; k++) xs[k] = jb + k * SUM_THREADS < c ? (uint32_t)__ldg(ti + jb + k * SUM_THREADS) ^ 0x80000000u : 0u;
#pragma unroll
      for (int k = 0; k < U; k++) {
        const uint32_t j = min(jb + k * SUM_THREADS, c - 1);   // a zero past the end multiplies any valid weight
        wide.mac(Fr::load_nc(w + (uint64_t)j * 8), xs[k]);
      }
    }
    acc = wide.to_fr();
  } else {
    for (uint32_t j = threadIdx.x; j < c; j += SUM_THREADS) {
      Fr v = Fr::load_nc(reinterpret_cast<const uint32_t*>(t) + (o * c + j) * 8);
      acc = fe_add(acc, fe_mul(v, Fr::load_nc(w + (uint64_t)j * 8)));
    }
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) {
    if (FROM_I32) acc = fe_sub(acc, Fr::load_nc(corr));
    acc.store(out + o * 8);
  }
}

void eq_weights_async(grape_ctx* ctx, const void* d_x, uint32_t nv, uint32_t c, void* d_w) {
  if (c == 0) return;
  k_eq_weights<<<ew_blocks(ctx, c), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_x, nv, c, (uint32_t*)d_w);
  ctx->launches += 1;
}

// ---- host-side launch helpers shared with the provers ---------------------------------------
// d_out = sum of n elements.  Uses its own arena allocation for the per-block partial sums.
int fr_sum_async(grape_ctx* ctx, const void* d_in, uint64_t n, void* d_out) {
  uint32_t blocks = ew_blocks(ctx, n);
  if (blocks > 1024) blocks = 1024;
  void* scratch;
  int rc = arena_alloc(ctx, (size_t)blocks * 32, &scratch);
  if (rc) return rc;
  k_sum_partial<<<blocks, SUM_THREADS, 0, ctx->stream>>>((const uint32_t*)d_in, n, (uint32_t*)scratch);
  k_sum_partial<<<1, SUM_THREADS, 0, ctx->stream>>>((const uint32_t*)scratch, blocks, (uint32_t*)d_out);
  ctx->launches += 2;
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

// Folds axis c of the [other][c][gap] view of d_t with challenges d_x[0..log2ceil(c)) into d_out
// ([other][gap]).  d_out must not alias d_t.  scratch_off: bytes of the arena the caller already uses.
template <bool FROM_I32>
int fold_axis_async(grape_ctx* ctx, const void* d_t, uint64_t ntot, const void* d_x, uint32_t c,
                    uint64_t gap, void* d_out) {
  if (c == 0 || gap == 0 || ntot % ((uint64_t)c * gap) != 0)
    return fail(ctx, GRAPE_ERR_INVALID, "fold: size is not a multiple of c*gap");
  const uint64_t other = ntot / ((uint64_t)c * gap);
  const uint64_t n_out = other * gap;
  const uint32_t nv = log2ceil(c);
  // A long innermost axis with few rows (a full evaluation of a big tensor is one row) would run in
  // `other` blocks: fold its low variables first, as rows of c_lo elements, then the short rest.
  if (gap == 1 && other < (uint64_t)ctx->sm_count * 4 && c >= 8192) {
    uint32_t lo_bits = nv / 2, tz = 0;
    while (tz < 31 && ((c >> tz) & 1u) == 0) tz++;
    if (lo_bits > tz) lo_bits = tz;
    if (lo_bits >= 6) {
      const uint32_t c_lo = 1u << lo_bits, c_hi = c >> lo_bits;
      void* tmp = nullptr;
      int rc0 = arena_alloc(ctx, (size_t)other * c_hi * 32, &tmp);
      if (rc0) return rc0;
      rc0 = fold_axis_async<FROM_I32>(ctx, d_t, ntot, d_x, c_lo, 1, tmp);
      if (rc0) return rc0;
      return fold_axis_async<false>(ctx, tmp, other * c_hi, reinterpret_cast<const uint32_t*>(d_x) + (size_t)lo_bits * 8,
                                    c_hi, 1, d_out);
    }
  }
  // work area: eq weights (c) + slice partials
  // staged kernel: int32 source, tensor 16-byte aligned, the tile width (512, 256 or 128 columns) divides gap
  int cpt = 0;
  if (FROM_I32 && gap > 1 && (reinterpret_cast<uintptr_t>(d_t) & 15) == 0) {
    if (gap % (4 * FOLD_THREADS) == 0) cpt = 4;
    else if (gap % (2 * FOLD_THREADS) == 0) cpt = 2;
    else if (gap % FOLD_THREADS == 0 && gap % 4 == 0) cpt = 1;
  }
  const uint64_t n_threads = cpt ? n_out / cpt : n_out;
  uint32_t n_slices = 1;
  if (gap > 1) {
    // Split the folded axis so that the grid fills the blocks the GPU can hold at once without
    // spilling a few blocks into one more wave (896 blocks on room for 444 run as three waves).
    int per_sm = 0;
    cudaError_t oe;
    if (cpt == 4) {
      GRAPE_CUDA_TRY(ctx, cudaFuncSetAttribute(k_fold_axis_i32_staged<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               StageLayout<4>::SMEM_BYTES));
      oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_fold_axis_i32_staged<4>, FOLD_THREADS,
                                                         StageLayout<4>::SMEM_BYTES);
    } else if (cpt == 2) {
      oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_fold_axis_i32_staged<2>, FOLD_THREADS,
                                                         StageLayout<2>::SMEM_BYTES);
    } else if (cpt == 1) {
      oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_fold_axis_i32_staged<1>, FOLD_THREADS,
                                                         StageLayout<1>::SMEM_BYTES);
    } else {
      oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_fold_axis<FROM_I32>, FOLD_THREADS, 0);
    }
    if (oe != cudaSuccess || per_sm < 1) per_sm = 4;
    const uint64_t room = (uint64_t)ctx->sm_count * per_sm;
    const uint64_t out_blocks = (n_threads + FOLD_THREADS - 1) / FOLD_THREADS;
    if (out_blocks < room) n_slices = (uint32_t)std::min<uint64_t>(room / out_blocks, (c + 15) / 16);
    if (n_slices < 1) n_slices = 1;
  }
  size_t w_bytes = ((size_t)c * 32 + 255) & ~size_t(255);
  size_t p_bytes = n_slices > 1 ? (size_t)n_slices * n_out * 32 : 0;
  void* d_work = nullptr;
  int arc = arena_alloc(ctx, w_bytes + p_bytes, &d_work);
  if (arc) return arc;
  uint32_t* w = reinterpret_cast<uint32_t*>(d_work);
  uint32_t* partial = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(d_work) + w_bytes);
  k_eq_weights<<<ew_blocks(ctx, c), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_x, nv, c, w);
  ctx->launches += 1;
  uint32_t* corr = nullptr;
  const uint32_t slice_len = gap == 1 ? c : (c + n_slices - 1) / n_slices;
  if (FROM_I32) {
    int crc = arena_alloc_t(ctx, (size_t)n_slices * 8 + 8, &corr);
    if (crc) return crc;
    k_bias_correction<<<gap == 1 ? 1 : n_slices, SUM_THREADS, 0, ctx->stream>>>(w, c, slice_len, corr);
    ctx->launches += 1;
  }
  if (gap == 1) {
    if (other > 0x7fffffffull) return fail(ctx, GRAPE_ERR_LIMIT, "fold: too many rows");
    k_fold_inner<FROM_I32><<<(uint32_t)other, SUM_THREADS, 0, ctx->stream>>>(d_t, w, c, (uint32_t*)d_out, corr);
    ctx->launches += 1;
  } else {
    dim3 grid((uint32_t)((n_threads + FOLD_THREADS - 1) / FOLD_THREADS), n_slices);
    uint32_t* fold_dst = n_slices > 1 ? partial : (uint32_t*)d_out;
    {
      ProfScope prof(ctx);
      const int32_t* ti = reinterpret_cast<const int32_t*>(d_t);
      if (cpt == 4) {
        k_fold_axis_i32_staged<4><<<grid, FOLD_THREADS, StageLayout<4>::SMEM_BYTES, ctx->stream>>>(
            ti, w, c, gap, n_out, slice_len, fold_dst, corr, ctx->d_status);
      } else if (cpt == 2) {
        k_fold_axis_i32_staged<2><<<grid, FOLD_THREADS, StageLayout<2>::SMEM_BYTES, ctx->stream>>>(
            ti, w, c, gap, n_out, slice_len, fold_dst, corr, ctx->d_status);
      } else if (cpt == 1) {
        k_fold_axis_i32_staged<1><<<grid, FOLD_THREADS, StageLayout<1>::SMEM_BYTES, ctx->stream>>>(
            ti, w, c, gap, n_out, slice_len, fold_dst, corr, ctx->d_status);
      } else {
        k_fold_axis<FROM_I32><<<grid, FOLD_THREADS, 0, ctx->stream>>>(d_t, w, c, gap, n_out, slice_len, fold_dst, corr);
      }
    }
    ctx->launches += 1;
    if (n_slices > 1) {
      k_sum_slices<<<ew_blocks(ctx, n_out), EW_THREADS, 0, ctx->stream>>>(partial, n_slices, n_out, (uint32_t*)d_out);
      ctx->launches += 1;
    }
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

template int fold_axis_async<false>(grape_ctx*, const void*, uint64_t, const void*, uint32_t, uint64_t, void*);
template int fold_axis_async<true>(grape_ctx*, const void*, uint64_t, const void*, uint32_t, uint64_t, void*);

}  // namespace grape

using namespace grape;

#define CHECK_CTX(ctx) if (!(ctx)) return GRAPE_ERR_INVALID
#define LAUNCH_DONE(ctx, k) do { (ctx)->launches += (k); GRAPE_CUDA_TRY((ctx), cudaGetLastError()); return GRAPE_OK; } while (0)

extern "C" int grape_fr_from_i32(grape_ctx* ctx, const int32_t* d_in, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_from_i32<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(d_in, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_from_u32(grape_ctx* ctx, const uint32_t* d_in, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_from_u32<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(d_in, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_to_mont(grape_ctx* ctx, void* d_t, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_to_mont<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((uint32_t*)d_t, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_from_mont(grape_ctx* ctx, void* d_t, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_from_mont<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((uint32_t*)d_t, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_add(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_binary<0, Fr><<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_sub(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_binary<1, Fr><<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_mul(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_binary<2, Fr><<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
// Diagnostics: the same three operations over the base field Fp (used by the curve arithmetic).
extern "C" int grape_fp_binary(grape_ctx* ctx, int op, const void* d_a, const void* d_b, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  uint32_t g = ew_blocks(ctx, n);
  if (op == 0) k_binary<0, Fp><<<g, EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  else if (op == 1) k_binary<1, Fp><<<g, EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  else if (op == 2) k_binary<2, Fp><<<g, EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  else return fail(ctx, GRAPE_ERR_INVALID, "fp_binary: op must be 0 (add), 1 (sub) or 2 (mul)");
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_scale(grape_ctx* ctx, const void* d_a, const void* d_scalar, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_broadcast<1><<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_scalar, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_add_scalar(grape_ctx* ctx, const void* d_a, const void* d_scalar, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_broadcast<0><<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_scalar, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_axpy(grape_ctx* ctx, const void* d_a, const void* d_scalar, const void* d_b, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return GRAPE_OK;
  k_axpy<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_a, (const uint32_t*)d_scalar, (const uint32_t*)d_b, (uint32_t*)d_out, n);
  LAUNCH_DONE(ctx, 1);
}
namespace grape {
// out[i] = 1 / (in[i] + shift); takes its prefix-product scratch from the arena without resetting it.
int fr_inverse_async(grape_ctx* ctx, const void* d_in, const void* d_shift, void* d_out, uint64_t n) {
  if (n == 0) return GRAPE_OK;
  void* scratch;
  int rc = arena_alloc(ctx, n * 32, &scratch);
  if (rc) return rc;
  // about 96 elements per thread once the tensor is large, at least one block per SM
  uint64_t threads = n / 96;
  uint64_t min_threads = (uint64_t)ctx->sm_count * 128;
  if (threads < min_threads) threads = std::min<uint64_t>(n, min_threads);
  uint32_t blocks = (uint32_t)((threads + 127) / 128);
  k_batch_inverse<<<blocks, 128, 0, ctx->stream>>>((const uint32_t*)d_in, (const uint32_t*)d_shift, (uint32_t*)d_out, (uint32_t*)scratch, n);
  ctx->launches += 1;
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}
}  // namespace grape
extern "C" int grape_fr_inverse(grape_ctx* ctx, const void* d_in, const void* d_shift, void* d_out, uint64_t n) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  arena_reset(ctx);
  return fr_inverse_async(ctx, d_in, d_shift, d_out, n);
}
extern "C" int grape_pad_i32(grape_ctx* ctx, const int32_t* d_in, int32_t* d_out, uint32_t n, uint32_t pad_n, uint64_t pad_size) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (pad_size == 0) return GRAPE_OK;
  if (n == 0 || pad_n < n) return fail(ctx, GRAPE_ERR_INVALID, "pad: need 0 < n <= pad_n");
  k_pad_i32<<<ew_blocks(ctx, pad_size), EW_THREADS, 0, ctx->stream>>>(d_in, d_out, n, pad_n, pad_size);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_pad(grape_ctx* ctx, const void* d_in, void* d_out, uint32_t n, uint32_t pad_n, uint64_t pad_size, const void* d_pad_value) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (pad_size == 0) return GRAPE_OK;
  if (n == 0 || pad_n < n) return fail(ctx, GRAPE_ERR_INVALID, "pad: need 0 < n <= pad_n");
  k_pad_fr<<<ew_blocks(ctx, pad_size), EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_in, (uint32_t*)d_out, n, pad_n, pad_size, (const uint32_t*)d_pad_value);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_sum(grape_ctx* ctx, const void* d_in, uint64_t n, void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (n == 0) return grape_dev_zero(ctx, d_out, 32);
  arena_reset(ctx);
  return fr_sum_async(ctx, d_in, n, d_out);
}
extern "C" int grape_fr_rowsum(grape_ctx* ctx, const void* d_in, void* d_out, uint64_t rows, uint32_t dim) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (rows == 0 || dim == 0) return GRAPE_OK;
  uint64_t threads = rows * 32;
  uint32_t blocks = ew_blocks(ctx, threads);
  k_rowsum_broadcast<<<blocks, EW_THREADS, 0, ctx->stream>>>((const uint32_t*)d_in, (uint32_t*)d_out, rows, dim);
  LAUNCH_DONE(ctx, 1);
}
extern "C" int grape_fr_fold(grape_ctx* ctx, const void* d_t, uint64_t ntot, const void* d_x, uint32_t c, uint64_t gap, void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (c == 0 || gap == 0) return fail(ctx, GRAPE_ERR_INVALID, "fold: c and gap must be positive");
  arena_reset(ctx);
  return fold_axis_async<false>(ctx, d_t, ntot, d_x, c, gap, d_out);
}
extern "C" int grape_fold_i32(grape_ctx* ctx, const int32_t* d_t, uint64_t ntot, const void* d_x, uint32_t c, uint64_t gap, void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  CHECK_CTX(ctx);
  if (c == 0 || gap == 0) return fail(ctx, GRAPE_ERR_INVALID, "fold: c and gap must be positive");
  arena_reset(ctx);
  return fold_axis_async<true>(ctx, d_t, ntot, d_x, c, gap, d_out);
}
