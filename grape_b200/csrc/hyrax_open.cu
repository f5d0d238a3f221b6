// Hyrax opening (the prover side of the evaluation proof).
//
// Replaces Hyrax::open (src/Hyrax.cu:237-305) and what it calls: single_commit (:176-185), the
// row / layer / inner folds (FrTensor::partial_eval), z = c*x + d, and the host-side scalar
// multiplication com_ad = <eq, d> * G (libff, :286-291), which here is one small kernel.
// The input tensor is left intact (the reference folds it in place and destroys it).
#include <algorithm>
#include <vector>

#include <cstring>

#include "ctx.cuh"
#include "curve.cuh"
#include "hostfr.hpp"

namespace grape {

template <bool FROM_I32>
int fold_axis_async(grape_ctx* ctx, const void* d_t, uint64_t ntot, const void* d_x, uint32_t c,
                    uint64_t gap, void* d_out);
int commit_fr_async(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size, uint32_t wd,
                    void* d_out);

// The context's SplitMix64 stream evaluated in parallel: the state after k steps is
// state0 + k * GOLDEN, so draw i (eight 64-bit outputs: four low words, four high words, reduced
// mod r as lo + hi * 2^256) needs no sequential dependency.  Same values as rng_next_fr on the host.
__device__ __forceinline__ uint64_t splitmix_at(uint64_t state0, uint64_t k) {
  uint64_t z = state0 + k * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__global__ void k_rng_fr(uint64_t state0, uint64_t n, uint32_t* __restrict__ out) {
  // 2^128 in Montgomery form; the 512 random bits are folded in four 128-bit pieces so that every
  // value entering a multiplication is far below the modulus' size limit
  const uint32_t t128[8] = {0xef8cfeb9u, 0xb075da81u, 0xa5b6cd8cu, 0xa7f12accu,
                            0x7957bf7bu, 0x32c47504u, 0x48ffa25eu, 0x03d581d7u};
  Fr T;
#pragma unroll
  for (int k = 0; k < 8; k++) T.v[k] = t128[k];
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    Fr acc = Fr::zero();
#pragma unroll
    for (int piece = 3; piece >= 0; piece--) {   // most significant 128 bits first
      uint64_t a = splitmix_at(state0, 8 * i + 1 + 2 * piece), b = splitmix_at(state0, 8 * i + 2 + 2 * piece);
      Fr c = Fr::zero();
      c.v[0] = (uint32_t)a;
      c.v[1] = (uint32_t)(a >> 32);
      c.v[2] = (uint32_t)b;
      c.v[3] = (uint32_t)(b >> 32);
      acc = fe_add(fe_mul(acc, T), fe_to_mont(c));
    }
    acc.store(out + i * 8);
  }
}

// The same vector from the ChaCha20 stream: element i is block `position0 + i` (64 bytes = 512 bits,
// reduced mod r as four 128-bit pieces).  Same values as rng_draw_fr on the host.
__global__ void k_rng_fr_chacha(RngKey key, uint64_t position0, uint64_t n, uint32_t* __restrict__ out) {
  const uint32_t t128[8] = {0xef8cfeb9u, 0xb075da81u, 0xa5b6cd8cu, 0xa7f12accu,
                            0x7957bf7bu, 0x32c47504u, 0x48ffa25eu, 0x03d581d7u};
  Fr T;
#pragma unroll
  for (int k = 0; k < 8; k++) T.v[k] = t128[k];
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t blk[16];
    chacha20_block(key.k, position0 + i, blk);
    Fr acc = Fr::zero();
#pragma unroll
    for (int piece = 3; piece >= 0; piece--) {   // most significant 128 bits first
      Fr c = Fr::zero();
#pragma unroll
      for (int k = 0; k < 4; k++) c.v[k] = blk[4 * piece + k];
      acc = fe_add(fe_mul(acc, T), fe_to_mont(c));
    }
    acc.store(out + i * 8);
  }
}

// The opening's second commitment is [sum_ad] * G for the protocol's fixed point G.  A double-and-add
// by one thread is 254 dependent doublings (1.8 ms with the rest of the GPU idle, as much as the
// whole rest of an opening), so G gets a fixed-base table of its own (16 windows of 16 bits, 32 MB, built
// once per context and per G) and the product becomes a one-element commitment: 16 table additions.
static int g_table_for(grape_ctx* ctx, const void* h_G_jacobian, const uint32_t* d_G, const grape_table** out) {
  if (ctx->g_table && memcmp(ctx->g_key, h_G_jacobian, sizeof ctx->g_key) == 0) {
    *out = ctx->g_table;
    return GRAPE_OK;
  }
  if (ctx->g_table) {
    GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    grape_table_destroy(ctx->g_table);
    ctx->g_table = nullptr;
  }
  grape_table* t = nullptr;
  int rc = grape_table_create(ctx, d_G, 1, 16, 16, &t);
  if (rc) return rc;
  ctx->g_table = t;
  memcpy(ctx->g_key, h_G_jacobian, sizeof ctx->g_key);
  *out = t;
  return GRAPE_OK;
}

}  // namespace grape

using namespace grape;

extern "C" int grape_hyrax_open(grape_ctx* ctx, const grape_table* table, const void* d_tensor, uint64_t size,
                                uint32_t N, uint32_t layer_num, const void* h_eval_point, uint32_t n_e,
                                const void* h_c, const void* h_G_jacobian, void* h_result, void* h_z,
                                void* h_com_d, void* h_com_ad) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !table || !d_tensor || !h_eval_point || !h_c || !h_G_jacobian || !h_result || !h_z || !h_com_d || !h_com_ad)
    return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (table->curve != 0) return fail(ctx, GRAPE_ERR_INVALID, "open: the opening protocol is built over BN254 only");
  if (N == 0 || layer_num == 0) return fail(ctx, GRAPE_ERR_INVALID, "open: zero dimension");
  if (size / N / GRAPE_COM_SCALE < layer_num)
    return fail(ctx, GRAPE_ERR_INVALID, "Size too small: size < N * com_scale * layer_num");
  const uint32_t pad_n = 1u << log2ceil(N);
  const uint32_t new_n = pad_n * GRAPE_COM_SCALE;
  const uint32_t wd = N * GRAPE_COM_SCALE;
  if (n_e != log2ceil(size)) return fail(ctx, GRAPE_ERR_INVALID, "open: eval_point.size() != Log2(size)");
  if (size % ((uint64_t)layer_num * wd) != 0) return fail(ctx, GRAPE_ERR_INVALID, "open: size is not layer_num * rows * N * 16");
  if (new_n > table->n_gens) return fail(ctx, GRAPE_ERR_INVALID, "open: the table has fewer generators than the padded row length");
  const uint32_t rows_per_layer = (uint32_t)(size / layer_num / wd);
  const HostFr* e = reinterpret_cast<const HostFr*>(h_eval_point);
  arena_reset(ctx);
  int rc;
  uint32_t *d_e, *d_cG, *d_d, *d_x1, *d_x, *d_xpad, *d_z, *d_small, *d_pts;
  if ((rc = arena_alloc_t(ctx, (size_t)n_e * 8 + 8, &d_e))) return rc;
  if ((rc = arena_alloc_t(ctx, 8 + 24 + 8, &d_cG))) return rc;       // c | G
  if ((rc = arena_alloc_t(ctx, (size_t)new_n * 8, &d_d))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)layer_num * wd * 8, &d_x1))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)new_n * 8, &d_x))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)new_n * 8, &d_xpad))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)new_n * 8, &d_z))) return rc;
  if ((rc = arena_alloc_t(ctx, 4 * 8, &d_small))) return rc;          // result | sum_ad | zero
  if ((rc = arena_alloc_t(ctx, 2 * 24 + 8, &d_pts))) return rc;       // com_d | com_ad
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_e, e, (size_t)n_e * 32, cudaMemcpyHostToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_cG, h_c, 32, cudaMemcpyHostToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(d_cG + 8, h_G_jacobian, 96, cudaMemcpyHostToDevice, ctx->stream));
  // blinding vector d from the context's random stream (reference: src/Hyrax.cu:253-256), generated on
  // the device; the host stream is advanced past the 8 words per element it consumed
  {
    const uint32_t rng_blocks = std::min<uint32_t>((new_n + 127) / 128, (uint32_t)ctx->sm_count * 8);
    if (ctx->rng.seeded) {
      k_rng_fr<<<rng_blocks, 128, 0, ctx->stream>>>(ctx->rng.splitmix, new_n, d_d);
      ctx->rng.splitmix += (uint64_t)new_n * 8 * 0x9E3779B97F4A7C15ull;
    } else {
      k_rng_fr_chacha<<<rng_blocks, 128, 0, ctx->stream>>>(ctx->rng.key, ctx->rng.position, new_n, d_d);
      ctx->rng.position += new_n;
    }
    ctx->launches += 1;
  }
  // com_d = sum_i d_i G_i
  if ((rc = commit_fr_async(ctx, table, d_d, new_n, new_n, d_pts))) return rc;
  // x = tensor folded over the row variables, then over the layer variables
  if ((rc = fold_axis_async<false>(ctx, d_tensor, size, d_e + (size_t)log2ceil(wd) * 8, rows_per_layer, wd, d_x1))) return rc;
  if ((rc = fold_axis_async<false>(ctx, d_x1, (uint64_t)wd * layer_num, d_e + (size_t)log2ceil(size / layer_num) * 8,
                                   layer_num, wd, d_x))) return rc;
  const uint32_t* xp = d_x;
  if (pad_n != N) {
    GRAPE_CUDA_TRY(ctx, cudaMemsetAsync(d_small + 16, 0, 32, ctx->stream));
    if ((rc = grape_fr_pad(ctx, d_x, d_xpad, N, pad_n, new_n, d_small + 16))) return rc;
    xp = d_xpad;
  }
  // result = x~(e[0..log2 new_n)),  z = c*x + d,  sum_ad = d~(e[0..))
  if ((rc = fold_axis_async<false>(ctx, xp, new_n, d_e, new_n, 1, d_small))) return rc;
  if ((rc = grape_fr_axpy(ctx, xp, d_cG, d_d, d_z, new_n))) return rc;
  if ((rc = fold_axis_async<false>(ctx, d_d, new_n, d_e, new_n, 1, d_small + 8))) return rc;
  // com_ad = [sum_ad] * G
  const grape_table* g_table = nullptr;
  if ((rc = g_table_for(ctx, h_G_jacobian, d_cG + 8, &g_table))) return rc;
  if ((rc = commit_fr_async(ctx, g_table, d_small + 8, 1, 1, d_pts + 24))) return rc;
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_result, d_small, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_z, d_z, (size_t)new_n * 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_com_d, d_pts, 96, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(h_com_ad, d_pts + 24, 96, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return GRAPE_OK;
}

// ---- variable-base linear combination (verifier side) ------------------------------------------
namespace grape {
// partial[warp] = sum over the warp's points of s_i * P_i (double-and-add per point, shuffle tree)
__global__ void __launch_bounds__(128) k_lincomb(const uint32_t* __restrict__ points_jac, const uint32_t* __restrict__ scalars,
                                                  uint64_t n, Xyzz* __restrict__ partial) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  Xyzz acc = Xyzz::inf();
  if (i < n) {
    Jacobian j;
    j.x = Fp::load(points_jac + i * 24);
    j.y = Fp::load(points_jac + i * 24 + 8);
    j.z = Fp::load(points_jac + i * 24 + 16);
    Xyzz base = xyzz_from_jacobian(j);
    Fr s = fe_from_mont(Fr::load(scalars + i * 8));
    for (int w = 7; w >= 0; w--) {
      for (int b = 31; b >= 0; b--) {
        acc = xyzz_dbl(acc);
        if ((s.v[w] >> b) & 1u) xyzz_add(acc, base);
      }
    }
  }
#pragma unroll 1
  for (int off = 16; off > 0; off >>= 1) {
    Xyzz other = xyzz_shfl_down(acc, off);
    if ((threadIdx.x & 31) < off) xyzz_add(acc, other);
  }
  if ((threadIdx.x & 31) == 0) acc.store(partial + (i >> 5));
}

__global__ void k_lincomb_finish(const Xyzz* __restrict__ partial, uint32_t n_partial, uint32_t* __restrict__ out_jac) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  Xyzz acc = Xyzz::inf();
  for (uint32_t k = 0; k < n_partial; k++) xyzz_add(acc, Xyzz::load(partial + k));
  bool inf = acc.is_inf();
  Affine a = xyzz_to_affine(acc);
  store_jacobian_normalised(out_jac, a, inf);
}
}  // namespace grape

// out = sum_i s_i * P_i for arbitrary Jacobian points and Fr scalars in device memory (what the
// reference's verifier code does on the host with libff: host_partial_me<G1> and Fr * G1,
// include/ec_operation.cuh:37-55, test/HyraxTest.cu:96-125).  d_out: one normalised Jacobian record.
extern "C" int grape_g1_lincomb(grape_ctx* ctx, const void* d_points_jacobian, const void* d_scalars, uint64_t n,
                                void* d_out) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_out || (n && (!d_points_jacobian || !d_scalars))) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (n > (uint64_t(1) << 24)) return fail(ctx, GRAPE_ERR_LIMIT, "lincomb: at most 2^24 points");
  arena_reset(ctx);
  const uint32_t blocks = (uint32_t)std::max<uint64_t>((n + 127) / 128, 1);
  Xyzz* partial = nullptr;
  int rc = arena_alloc_t(ctx, (size_t)blocks * 4, &partial);
  if (rc) return rc;
  k_lincomb<<<blocks, 128, 0, ctx->stream>>>((const uint32_t*)d_points_jacobian, (const uint32_t*)d_scalars, n, partial);
  k_lincomb_finish<<<1, 32, 0, ctx->stream>>>(partial, blocks * 4, (uint32_t*)d_out);
  ctx->launches += 2;
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}
