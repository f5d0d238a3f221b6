// Sumcheck provers for matrix products, Hadamard products and claim batching.
//
// Replaces (paths inside the reference project):
//   sumcheck_kernel x2                          src/prove.cu:14-46
//   matmul_sumcheck_phase1 / phase2             src/prove.cu:49-117
//   eleMul_sumcheck                             src/prove.cu:119-172
//   prove_matmul / prove_eleMul / combine_claims  src/prove.cu:175-301
//
// How the work is organised here.  Every Fiat-Shamir-style challenge is an INPUT of these provers
// (the reference takes u and v as arguments too), so nothing the device does in round i+1 depends
// on the host's view of round i.  All rounds are therefore enqueued back to back on the stream:
// one fused kernel per round folds the tensors in place by the round's challenge and accumulates
// the few field sums the round polynomial needs (in registers, then warp shuffles, then one
// partial per block), a second tiny kernel adds the block partials into that round's slot of a
// device buffer.  After the last round the buffer comes back in ONE copy and the host assembles
// the round polynomials, runs the reference's p(0)+p(1)==claim checks and updates the claims.
// The reference instead materialises three coefficient tensors per round, folds each of them with
// log2 launches, reduces them with multi-pass sums and synchronises about twenty times per round.
#include <algorithm>
#include <cstring>
#include <vector>

#include "ctx.cuh"
#include "field.cuh"
#include "hostfr.hpp"

namespace grape {

// implemented in frtensor.cu
template <bool FROM_I32>
int fold_axis_async(grape_ctx* ctx, const void* d_t, uint64_t ntot, const void* d_x, uint32_t c,
                    uint64_t gap, void* d_out);

constexpr int RT = 256;  // threads per block of the round kernels

// Block-wide sum of NS field elements per thread -> dst[NS] (valid after return in thread 0 only).
template <int NS>
__device__ __forceinline__ void block_reduce_store(Fr (&acc)[NS], uint32_t* __restrict__ dst) {
  __shared__ Fr part[RT / 32][NS];
#pragma unroll
  for (int s = 0; s < NS; s++) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[s] = fe_add(acc[s], fe_shfl_down(acc[s], off));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; s++) part[warp][s] = acc[s];
  }
  __syncthreads();
  if (threadIdx.x < NS) {
    Fr v = part[0][threadIdx.x];
    for (int w = 1; w < RT / 32; w++) v = fe_add(v, part[w][threadIdx.x]);
    v.store(dst + threadIdx.x * 8);
  }
}

// sums[slot][s] = sum over blocks of partial[block][s]
template <int NS>
__global__ void __launch_bounds__(RT) k_reduce_partials(const uint32_t* __restrict__ partial, uint32_t n_blocks,
                                                        uint32_t* __restrict__ dst) {
  Fr acc[NS];
#pragma unroll
  for (int s = 0; s < NS; s++) acc[s] = Fr::zero();
  for (uint32_t b = threadIdx.x; b < n_blocks; b += RT) {
#pragma unroll
    for (int s = 0; s < NS; s++) acc[s] = fe_add(acc[s], Fr::load_nc(partial + ((uint64_t)b * NS + s) * 8));
  }
  block_reduce_store<NS>(acc, dst);
}

// Weight of pair g: (whi ? whi[g / lo_len] : 1) * (wlo ? wlo[g % lo_len] : 1)
struct PairWeights {
  const uint32_t* whi;
  const uint32_t* wlo;
  uint32_t lo_len;
};

// One round over two tensors (reference: the five-pointer sumcheck_kernel, src/prove.cu:29-46, plus
// the folds and sums of its three outputs).  For every pair (g, g + out_size):
//   A(t) = Ab + t*Aa, B(t) = Bb + t*Ba,  accumulate  w*Ab*Bb, w*(Aa*Bb + Ab*Ba), w*Aa*Ba,
//   then A[g] <- Ab + v*Aa, B[g] <- Bb + v*Ba.   A pair whose upper half lies past in_size pairs with zero.
template <bool WHI, bool WLO>
__global__ void __launch_bounds__(RT)
k_round_two(uint32_t* __restrict__ A, uint32_t* __restrict__ B, uint64_t in_size, uint64_t out_size,
            const uint32_t* __restrict__ v, PairWeights pw, uint32_t* __restrict__ partial) {
  const Fr vv = Fr::load_nc(v);
  Fr acc[3] = {Fr::zero(), Fr::zero(), Fr::zero()};
  for (uint64_t g = (uint64_t)blockIdx.x * RT + threadIdx.x; g < out_size; g += (uint64_t)gridDim.x * RT) {
    Fr Ab = Fr::load(A + g * 8), Bb = Fr::load(B + g * 8);
    Fr Aa, Ba;
    if (g + out_size < in_size) {
      Aa = fe_sub(Fr::load(A + (g + out_size) * 8), Ab);
      Ba = fe_sub(Fr::load(B + (g + out_size) * 8), Bb);
    } else {
      Aa = fe_neg(Ab);
      Ba = fe_neg(Bb);
    }
    fe_add(Ab, fe_mul(Aa, vv)).store(A + g * 8);
    fe_add(Bb, fe_mul(Ba, vv)).store(B + g * 8);
    Fr wa = Aa, wb = Ab;
    if (WHI || WLO) {
      Fr w;
      if (WHI && WLO) w = fe_mul(Fr::load_nc(pw.whi + (g / pw.lo_len) * 8), Fr::load_nc(pw.wlo + (g % pw.lo_len) * 8));
      else if (WHI) w = Fr::load_nc(pw.whi + (g / pw.lo_len) * 8);
      else w = Fr::load_nc(pw.wlo + (g % pw.lo_len) * 8);
      wa = fe_mul(Aa, w);
      wb = fe_mul(Ab, w);
    }
    Fr c0 = fe_mul(wb, Bb);
    Fr c2 = fe_mul(wa, Ba);
    Fr mid = fe_mul(fe_add(wa, wb), fe_add(Ba, Bb));  // Karatsuba: cross term = mid - c0 - c2
    acc[0] = fe_add(acc[0], c0);
    acc[1] = fe_add(acc[1], fe_sub(fe_sub(mid, c0), c2));
    acc[2] = fe_add(acc[2], c2);
  }
  block_reduce_store<3>(acc, partial + (uint64_t)blockIdx.x * 3 * 8);
}

// The last rounds of an unweighted two-tensor sumcheck in ONE launch: once the tensors are short
// (a few thousand elements) a round is far shorter than a kernel launch, so a single block runs
// round after round with a block barrier in between.  Round r folds by v[v_first - r] and leaves its
// three sums in sums[r]; sizes follow the reference's rule (in_size, then halving powers of two).
constexpr uint32_t TAIL_MAX = 8192;
__global__ void __launch_bounds__(RT)
k_rounds_tail(uint32_t* __restrict__ A, uint32_t* __restrict__ B, uint64_t in_size, uint64_t out_size, uint32_t n_rounds,
              const uint32_t* __restrict__ v, uint32_t v_first, uint32_t* __restrict__ sums) {
  for (uint32_t r = 0; r < n_rounds; r++) {
    const Fr vv = Fr::load_nc(v + (uint64_t)(v_first - r) * 8);
    Fr acc[3] = {Fr::zero(), Fr::zero(), Fr::zero()};
    for (uint64_t g = threadIdx.x; g < out_size; g += RT) {
      Fr Ab = Fr::load(A + g * 8), Bb = Fr::load(B + g * 8);
      Fr Aa, Ba;
      if (g + out_size < in_size) {
        Aa = fe_sub(Fr::load(A + (g + out_size) * 8), Ab);
        Ba = fe_sub(Fr::load(B + (g + out_size) * 8), Bb);
      } else {
        Aa = fe_neg(Ab);
        Ba = fe_neg(Bb);
      }
      fe_add(Ab, fe_mul(Aa, vv)).store(A + g * 8);
      fe_add(Bb, fe_mul(Ba, vv)).store(B + g * 8);
      Fr c0 = fe_mul(Ab, Bb);
      Fr c2 = fe_mul(Aa, Ba);
      Fr mid = fe_mul(fe_add(Aa, Ab), fe_add(Ba, Bb));
      acc[0] = fe_add(acc[0], c0);
      acc[1] = fe_add(acc[1], fe_sub(fe_sub(mid, c0), c2));
      acc[2] = fe_add(acc[2], c2);
    }
    block_reduce_store<3>(acc, sums + (uint64_t)r * 3 * 8);
    __syncthreads();  // the folded values and the shared scratch are settled before the next round
    in_size = out_size;
    out_size /= 2;
  }
}

// One round over one tensor with J weight sets (combine_claims; reference: the three-pointer
// sumcheck_kernel, src/prove.cu:14-27, plus two full evaluations per claim).  For every pair:
//   X(t) = Xb + t*Xa; per claim j accumulate w_j*Xb and w_j*Xa with w_j = whi_j[g >> lo_bits] * wlo_j[g & mask];
//   then X[g] <- Xb + v*Xa.
constexpr int MAX_CLAIMS = 4;
struct ClaimWeights {
  const uint32_t* whi[MAX_CLAIMS];
  const uint32_t* wlo[MAX_CLAIMS];
  uint32_t lo_bits;
};

template <int J>
__global__ void __launch_bounds__(RT)
k_round_one(uint32_t* __restrict__ X, uint64_t out_size, const uint32_t* __restrict__ v, ClaimWeights cw,
            uint32_t* __restrict__ partial) {
  const Fr vv = Fr::load_nc(v);
  Fr acc[2 * J];
#pragma unroll
  for (int s = 0; s < 2 * J; s++) acc[s] = Fr::zero();
  const uint64_t mask = (uint64_t(1) << cw.lo_bits) - 1;
  for (uint64_t g = (uint64_t)blockIdx.x * RT + threadIdx.x; g < out_size; g += (uint64_t)gridDim.x * RT) {
    Fr Xb = Fr::load(X + g * 8);
    Fr Xa = fe_sub(Fr::load(X + (g + out_size) * 8), Xb);
    fe_add(Xb, fe_mul(Xa, vv)).store(X + g * 8);
#pragma unroll
    for (int j = 0; j < J; j++) {
      Fr w = fe_mul(Fr::load_nc(cw.whi[j] + (g >> cw.lo_bits) * 8), Fr::load_nc(cw.wlo[j] + (g & mask) * 8));
      acc[2 * j] = fe_add(acc[2 * j], fe_mul(w, Xb));
      acc[2 * j + 1] = fe_add(acc[2 * j + 1], fe_mul(w, Xa));
    }
  }
  block_reduce_store<2 * J>(acc, partial + (uint64_t)blockIdx.x * 2 * J * 8);
}

// implemented in frtensor.cu: w[j] = prod_k (bit_k(j) ? x_k : 1 - x_k), j < c
void eq_weights_async(grape_ctx* ctx, const void* d_x, uint32_t nv, uint32_t c, void* d_w);

static uint32_t round_blocks(const grape_ctx* ctx, uint64_t out_size) {
  uint64_t b = (out_size + RT - 1) / RT;
  uint64_t cap = (uint64_t)ctx->sm_count * 4;
  if (b > cap) b = cap;
  return (uint32_t)std::max<uint64_t>(b, 1);
}

// ---- host-side polynomial helpers (degree <= 3) ---------------------------------------------
struct Poly {
  HostFr c[4];
  int n;  // number of coefficients
};
static Poly poly_mul_eq(const HostFr q[3], const HostFr& u, const HostFr& scale) {
  // q(t) * ((1-u) + (2u-1) t) * scale
  HostFr e0 = fr_mul(fr_sub(fr_one(), u), scale);
  HostFr e1 = fr_mul(fr_sub(fr_add(u, u), fr_one()), scale);
  Poly p;
  p.n = 4;
  p.c[0] = fr_mul(q[0], e0);
  p.c[1] = fr_add(fr_mul(q[1], e0), fr_mul(q[0], e1));
  p.c[2] = fr_add(fr_mul(q[2], e0), fr_mul(q[1], e1));
  p.c[3] = fr_mul(q[2], e1);
  return p;
}
static HostFr poly_at01(const Poly& p) {
  HostFr s = p.c[0];
  for (int i = 0; i < p.n; i++) s = fr_add(s, p.c[i]);
  return s;
}
static HostFr poly_eval(const Poly& p, const HostFr& x) {
  HostFr acc = p.c[p.n - 1];
  for (int i = p.n - 2; i >= 0; i--) acc = fr_add(fr_mul(acc, x), p.c[i]);
  return acc;
}

static void emit(std::vector<HostFr>* transcript, const Poly& p) {
  if (!transcript) return;
  for (int i = 0; i < 4; i++) transcript->push_back(i < p.n ? p.c[i] : fr_zero());
}

// Describes one enqueued round for the host pass that follows.
struct RoundInfo {
  bool with_eq;   // round polynomial carries the eq(u_now) factor (degree 3) and updates E
  HostFr u_now, v_now;
};

static int upload_fr(grape_ctx* ctx, const HostFr* h, size_t n, uint32_t** d) {
  int rc = arena_alloc_t(ctx, n * 8 + 8, d);
  if (rc) return rc;
  if (n) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(*d, h, n * 32, cudaMemcpyHostToDevice, ctx->stream));
  return GRAPE_OK;
}

// Runs the host pass over the sums of all rounds of a two-tensor sumcheck.
static int finish_two(grape_ctx* ctx, const std::vector<RoundInfo>& rounds, const uint32_t* d_sums,
                      const uint32_t* d_A, const uint32_t* d_B, HostFr* claim, HostFr* out_claims,
                      std::vector<HostFr>* transcript, const char* what) {
  std::vector<HostFr> sums(rounds.size() * 3 + 2);
  if (!rounds.empty())
    GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(sums.data(), d_sums, rounds.size() * 3 * 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&sums[rounds.size() * 3], d_A, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&sums[rounds.size() * 3 + 1], d_B, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  HostFr E = fr_one();
  for (size_t i = 0; i < rounds.size(); i++) {
    const HostFr* q = &sums[i * 3];
    Poly p;
    if (rounds[i].with_eq) {
      p = poly_mul_eq(q, rounds[i].u_now, E);
    } else {
      p.n = 3;
      for (int k = 0; k < 3; k++) p.c[k] = fr_mul(q[k], E);
    }
    emit(transcript, p);
    if (poly_at01(p) != *claim)
      return fail(ctx, GRAPE_ERR_CHECK, std::string(what) + ": claim != p(0) + p(1) in round " + std::to_string(i));
    *claim = poly_eval(p, rounds[i].v_now);
    if (rounds[i].with_eq) E = fr_mul(E, fr_eq2(rounds[i].u_now, rounds[i].v_now));
  }
  out_claims[0] = sums[rounds.size() * 3];
  out_claims[1] = sums[rounds.size() * 3 + 1];
  if (fr_mul(fr_mul(out_claims[0], out_claims[1]), E) != *claim)
    return fail(ctx, GRAPE_ERR_CHECK, std::string(what) + ": final identity A*B*eq != claim");
  return GRAPE_OK;
}

template <bool WHI, bool WLO>
static void launch_round_two(grape_ctx* ctx, uint32_t* A, uint32_t* B, uint64_t in_size, uint64_t out_size,
                             const uint32_t* d_v, PairWeights pw, uint32_t* partial, uint32_t* sums_slot) {
  uint32_t blocks = round_blocks(ctx, out_size);
  k_round_two<WHI, WLO><<<blocks, RT, 0, ctx->stream>>>(A, B, in_size, out_size, d_v, pw, partial);
  k_reduce_partials<3><<<1, RT, 0, ctx->stream>>>(partial, blocks, sums_slot);
  ctx->launches += 2;
}

}  // namespace grape

namespace grape {

// Everything grape_prove_matmul enqueues before its host pass: the two axis folds and one fused
// kernel pair per round.  On return the stream holds all the work; `sums` gets three field
// elements per round and a_[0], b_[0] the fully folded values.
struct MatmulRun {
  uint32_t *d_u = nullptr, *d_v = nullptr, *a_ = nullptr, *b_ = nullptr, *partial = nullptr, *sums = nullptr, *wl = nullptr;
  uint32_t lL = 0, lK = 0, u_end = 0, v_end = 0;
  std::vector<RoundInfo> rounds;
};

template <bool FROM_I32 = false>
static int matmul_enqueue(grape_ctx* ctx, const void* d_A, const void* d_B, uint32_t L, uint32_t N, uint32_t M, uint32_t K,
                          const HostFr* u, uint32_t n_u, const HostFr* v, uint32_t n_v, MatmulRun& run) {
  if (!L || !N || !M || !K) return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul: zero dimension");
  const uint32_t lL = log2ceil(L), lN = log2ceil(N), lM = log2ceil(M), lK = log2ceil(K);
  if ((1u << lL) != L) return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul: L must be a power of two");
  const uint32_t u_end = log2ceil((uint64_t)L * N * M), v_end = log2ceil((uint64_t)L * K);
  if (n_u < u_end || n_u < lM + lN + lL || n_v < v_end || n_v < lK)
    return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul: challenge vectors too short");
  run.lL = lL;
  run.lK = lK;
  run.u_end = u_end;
  run.v_end = v_end;
  arena_reset(ctx);
  int rc;
  if ((rc = upload_fr(ctx, u, n_u, &run.d_u))) return rc;
  if ((rc = upload_fr(ctx, v, n_v, &run.d_v))) return rc;
  const uint64_t LK = (uint64_t)L * K;
  if ((rc = arena_alloc_t(ctx, LK * 8, &run.a_))) return rc;
  if ((rc = arena_alloc_t(ctx, LK * 8, &run.b_))) return rc;
  const uint32_t total_rounds = lL + lK;
  if ((rc = arena_alloc_t(ctx, (size_t)ctx->sm_count * 4 * 3 * 8 + 64, &run.partial))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)(total_rounds + 1) * 3 * 8, &run.sums))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)L * 8 + 8, &run.wl))) return rc;
  uint32_t *d_u = run.d_u, *d_v = run.d_v, *a_ = run.a_, *b_ = run.b_;
  // a_[l][k] = sum_n eq(u_N, n) A[l][n][k],  b_[l][k] = sum_m eq(u_M, m) B[l][m][k]
  if ((rc = fold_axis_async<FROM_I32>(ctx, d_A, (uint64_t)L * N * K, d_u + (size_t)lM * 8, N, K, a_))) return rc;
  if ((rc = fold_axis_async<FROM_I32>(ctx, d_B, (uint64_t)L * M * K, d_u, M, K, b_))) return rc;

  std::vector<RoundInfo>& rounds = run.rounds;
  uint64_t in_size = LK, out_size = LK / 2;
  const uint32_t u_l0 = u_end - lL;
  for (uint32_t i = 0; i < lL; i++) {  // phase 1: layer variables, top first
    const uint32_t rem_layers = (uint32_t)(out_size / K);
    eq_weights_async(ctx, d_u + (size_t)u_l0 * 8, log2ceil(rem_layers), rem_layers, run.wl);
    PairWeights pw{run.wl, nullptr, K};
    launch_round_two<true, false>(ctx, a_, b_, in_size, out_size, d_v + (size_t)(v_end - i - 1) * 8, pw, run.partial,
                                  run.sums + (size_t)rounds.size() * 3 * 8);
    rounds.push_back({true, u[u_end - i - 1], v[v_end - i - 1]});
    in_size = out_size;
    out_size /= 2;
  }
  in_size = K;
  out_size = lK ? (uint64_t(1) << (lK - 1)) : 0;
  for (uint32_t i = 0; i < lK; i++) {  // phase 2: inner-product variables, top first
    if (in_size <= TAIL_MAX) {  // all remaining rounds in one launch
      k_rounds_tail<<<1, RT, 0, ctx->stream>>>(a_, b_, in_size, out_size, lK - i, d_v, lK - i - 1,
                                               run.sums + (size_t)rounds.size() * 3 * 8);
      ctx->launches += 1;
      for (; i < lK; i++) rounds.push_back({false, fr_zero(), v[lK - i - 1]});
      break;
    }
    PairWeights pw{nullptr, nullptr, 1};
    launch_round_two<false, false>(ctx, a_, b_, in_size, out_size, d_v + (size_t)(lK - i - 1) * 8, pw, run.partial,
                                   run.sums + (size_t)rounds.size() * 3 * 8);
    rounds.push_back({false, fr_zero(), v[lK - i - 1]});
    in_size = out_size;
    out_size /= 2;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  return GRAPE_OK;
}

// Sharded finish: adds the per-rank round sums (mod r) and lays the per-rank folded values out as
// the two length-P vectors the last log2(P) rounds run over.  One block.
//   gathered: [P][stride] field elements, stride = 3 * local_rounds + 2
__global__ void __launch_bounds__(RT) k_gather_reduce(const uint32_t* __restrict__ gathered, uint32_t P,
                                                      uint32_t local_rounds, uint32_t* __restrict__ sums,
                                                      uint32_t* __restrict__ a_, uint32_t* __restrict__ b_) {
  const uint32_t stride = 3 * local_rounds + 2;
  for (uint32_t s = threadIdx.x; s < 3 * local_rounds; s += RT) {
    Fr acc = Fr::load_nc(gathered + (uint64_t)s * 8);
    for (uint32_t r = 1; r < P; r++) acc = fe_add(acc, Fr::load_nc(gathered + ((uint64_t)r * stride + s) * 8));
    acc.store(sums + (uint64_t)s * 8);
  }
  for (uint32_t r = threadIdx.x; r < P; r += RT) {
    Fr::load_nc(gathered + ((uint64_t)r * stride + 3 * local_rounds) * 8).store(a_ + (uint64_t)r * 8);
    Fr::load_nc(gathered + ((uint64_t)r * stride + 3 * local_rounds + 1) * 8).store(b_ + (uint64_t)r * 8);
  }
}

}  // namespace grape

using namespace grape;

// prove_matmul (src/prove.cu:175-210).  d_A = [L][N][K], d_B = [L][M][K] Fr tensors; both are
// consumed (left in an unspecified state) like the reference's in-place folds.
extern "C" int grape_prove_matmul(grape_ctx* ctx, void* d_A, void* d_B, uint32_t L, uint32_t N, uint32_t M,
                                  uint32_t K, const void* h_u, uint32_t n_u, const void* h_v, uint32_t n_v,
                                  void* h_claim, void* h_out_claims, void* h_transcript,
                                  uint32_t transcript_capacity, uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_A || !d_B || !h_u || !h_v || !h_claim || !h_out_claims) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  MatmulRun run;
  int rc = matmul_enqueue(ctx, d_A, d_B, L, N, M, K, reinterpret_cast<const HostFr*>(h_u), n_u,
                          reinterpret_cast<const HostFr*>(h_v), n_v, run);
  if (rc) return rc;
  std::vector<HostFr> transcript;
  rc = finish_two(ctx, run.rounds, run.sums, run.a_, run.b_, reinterpret_cast<HostFr*>(h_claim),
                  reinterpret_cast<HostFr*>(h_out_claims), &transcript, "prove_matmul");
  if (n_rounds) *n_rounds = (uint32_t)(transcript.size() / 4);
  if (h_transcript) {
    size_t n = std::min<size_t>(transcript.size(), (size_t)transcript_capacity * 4);
    memcpy(h_transcript, transcript.data(), n * 32);
  }
  return rc;
}

// prove_matmul on the int32 tensors the reference builds its FrTensors from (FrTensor(uint, int*),
// src/fr-tensor.cu:30-46,190-197, immediately before every prove_matmul of its drivers).  Same
// claims and transcript as converting to Fr first and calling grape_prove_matmul; the two axis
// folds, which dominate the proof, then read 4 bytes per element instead of 32 and skip the field
// multiplication per element.  The inputs are left intact.
extern "C" int grape_prove_matmul_i32(grape_ctx* ctx, const int32_t* d_A, const int32_t* d_B, uint32_t L, uint32_t N,
                                      uint32_t M, uint32_t K, const void* h_u, uint32_t n_u, const void* h_v,
                                      uint32_t n_v, void* h_claim, void* h_out_claims, void* h_transcript,
                                      uint32_t transcript_capacity, uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_A || !d_B || !h_u || !h_v || !h_claim || !h_out_claims) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  MatmulRun run;
  int rc = matmul_enqueue<true>(ctx, d_A, d_B, L, N, M, K, reinterpret_cast<const HostFr*>(h_u), n_u,
                                reinterpret_cast<const HostFr*>(h_v), n_v, run);
  if (rc) return rc;
  std::vector<HostFr> transcript;
  rc = finish_two(ctx, run.rounds, run.sums, run.a_, run.b_, reinterpret_cast<HostFr*>(h_claim),
                  reinterpret_cast<HostFr*>(h_out_claims), &transcript, "prove_matmul");
  if (n_rounds) *n_rounds = (uint32_t)(transcript.size() / 4);
  if (h_transcript) {
    size_t n = std::min<size_t>(transcript.size(), (size_t)transcript_capacity * 4);
    memcpy(h_transcript, transcript.data(), n * 32);
  }
  return rc;
}

// ---- prove_matmul split over P provers --------------------------------------------------------
// The inner dimension is dealt to P = 2^p provers by residue class: prover r holds the columns
// k = k' * P + r of A and B as dense [L][N][K/P] and [L][M][K/P] tensors.  The reference folds the
// most significant variable first, so every round over the top log2(K) - p variables pairs elements
// that live on the same prover: each prover runs those rounds alone on its shard (all challenges
// are inputs) and produces per-round PARTIAL sums; the true round sums are the sums of the partials
// over the provers.  One exchange -- (3 * local_rounds + 2) field elements per prover, gathered to
// everyone -- replaces any per-round communication; the last p rounds run over the P gathered
// folded values.  The transcript is bit-identical to grape_prove_matmul on the unsharded tensors.
//
// Step 1 (every prover): enqueue the local rounds on the shard and leave, in d_part (device memory
// of this prover, (3 * local_rounds + 2) * 32 bytes), the partial sums followed by the shard's fully
// folded A and B values.  h_v_local is v without its lowest p entries.  Asynchronous on the
// context's stream; *local_rounds = log2(L) + log2ceil(K_local).
extern "C" int grape_prove_matmul_partial(grape_ctx* ctx, void* d_A_shard, void* d_B_shard, uint32_t L, uint32_t N,
                                          uint32_t M, uint32_t K_local, const void* h_u, uint32_t n_u,
                                          const void* h_v_local, uint32_t n_v_local, void* d_part,
                                          uint32_t* local_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_A_shard || !d_B_shard || !h_u || !h_v_local || !d_part)
    return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  MatmulRun run;
  int rc = matmul_enqueue(ctx, d_A_shard, d_B_shard, L, N, M, K_local, reinterpret_cast<const HostFr*>(h_u), n_u,
                          reinterpret_cast<const HostFr*>(h_v_local), n_v_local, run);
  if (rc) return rc;
  const size_t nr = run.rounds.size();
  char* out = reinterpret_cast<char*>(d_part);
  if (nr) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(out, run.sums, nr * 96, cudaMemcpyDeviceToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(out + nr * 96, run.a_, 32, cudaMemcpyDeviceToDevice, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(out + nr * 96 + 32, run.b_, 32, cudaMemcpyDeviceToDevice, ctx->stream));
  if (local_rounds) *local_rounds = (uint32_t)nr;
  return GRAPE_OK;
}

// Step 2 (any prover that holds the gathered buffer): d_gathered = the P provers' d_part buffers in
// rank order.  Reduces the partial sums on the device, runs the last log2(P) rounds over the
// gathered folded values, then the host pass of grape_prove_matmul (round checks, claims,
// transcript).  N, M, K are the full dimensions; h_u, h_v, h_claim as in grape_prove_matmul.
extern "C" int grape_prove_matmul_finish(grape_ctx* ctx, const void* d_gathered, uint32_t P, uint32_t L, uint32_t N,
                                         uint32_t M, uint32_t K, const void* h_u, uint32_t n_u, const void* h_v,
                                         uint32_t n_v, void* h_claim, void* h_out_claims, void* h_transcript,
                                         uint32_t transcript_capacity, uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_gathered || !h_u || !h_v || !h_claim || !h_out_claims) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (!P || !L || !N || !M || !K) return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul_finish: zero dimension");
  const uint32_t lP = log2ceil(P), lL = log2ceil(L), lK = log2ceil(K);
  if ((1u << lP) != P || (1u << lL) != L) return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul_finish: P and L must be powers of two");
  if (K % P != 0 || lK < lP) return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul_finish: P must divide K");
  const uint32_t u_end = log2ceil((uint64_t)L * N * M), v_end = log2ceil((uint64_t)L * K);
  if (n_u < u_end || n_v < v_end || n_v < lK)
    return fail(ctx, GRAPE_ERR_INVALID, "prove_matmul_finish: challenge vectors too short");
  const HostFr* u = reinterpret_cast<const HostFr*>(h_u);
  const HostFr* v = reinterpret_cast<const HostFr*>(h_v);
  const uint32_t local_rounds = lL + (lK - lP);
  arena_reset(ctx);
  uint32_t *d_v, *a_, *b_, *partial, *sums;
  int rc;
  if ((rc = upload_fr(ctx, v, n_v, &d_v))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)P * 8 + 8, &a_))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)P * 8 + 8, &b_))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)ctx->sm_count * 4 * 3 * 8 + 64, &partial))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)(lL + lK + 1) * 3 * 8, &sums))) return rc;
  k_gather_reduce<<<1, RT, 0, ctx->stream>>>(reinterpret_cast<const uint32_t*>(d_gathered), P, local_rounds, sums, a_, b_);
  ctx->launches += 1;
  std::vector<RoundInfo> rounds;
  for (uint32_t i = 0; i < lL; i++) rounds.push_back({true, u[u_end - i - 1], v[v_end - i - 1]});
  for (uint32_t i = 0; i < lK - lP; i++) rounds.push_back({false, fr_zero(), v[lK - i - 1]});
  uint64_t in_size = P, out_size = P / 2;
  for (uint32_t i = 0; i < lP; i++) {  // the variables that index the provers
    PairWeights pw{nullptr, nullptr, 1};
    launch_round_two<false, false>(ctx, a_, b_, in_size, out_size, d_v + (size_t)(lP - i - 1) * 8, pw, partial,
                                   sums + (size_t)rounds.size() * 3 * 8);
    rounds.push_back({false, fr_zero(), v[lP - i - 1]});
    in_size = out_size;
    out_size /= 2;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  std::vector<HostFr> transcript;
  rc = finish_two(ctx, rounds, sums, a_, b_, reinterpret_cast<HostFr*>(h_claim), reinterpret_cast<HostFr*>(h_out_claims),
                  &transcript, "prove_matmul (sharded)");
  if (n_rounds) *n_rounds = (uint32_t)(transcript.size() / 4);
  if (h_transcript) {
    size_t n = std::min<size_t>(transcript.size(), (size_t)transcript_capacity * 4);
    memcpy(h_transcript, transcript.data(), n * 32);
  }
  return rc;
}

// prove_eleMul (src/prove.cu:212-241 with eleMul_sumcheck :119-172).  A, B = [L*M][N] Fr tensors.
extern "C" int grape_prove_elemul(grape_ctx* ctx, void* d_A, void* d_B, uint32_t L, uint32_t M, uint32_t N,
                                  const void* h_u, uint32_t n_u, const void* h_v, uint32_t n_v, void* h_claim,
                                  void* h_out_claims, void* h_transcript, uint32_t transcript_capacity,
                                  uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_A || !d_B || !h_u || !h_v || !h_claim || !h_out_claims) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (!L || !N || !M) return fail(ctx, GRAPE_ERR_INVALID, "prove_eleMul: zero dimension");
  const uint64_t first_size = (uint64_t)L * M, size = first_size * N;
  if ((uint64_t(1) << log2ceil(first_size)) != first_size)
    return fail(ctx, GRAPE_ERR_INVALID, "eleMul_sumcheck: first_size is illegal");
  const uint32_t second_size = N;
  const uint32_t rounds_n = log2ceil(size), l_first = log2ceil(first_size), l_in = log2ceil(N);
  const uint32_t u_end = rounds_n, v_end = rounds_n;
  if (n_u < u_end || n_v < v_end) return fail(ctx, GRAPE_ERR_INVALID, "prove_eleMul: challenge vectors too short");
  const HostFr* u = reinterpret_cast<const HostFr*>(h_u);
  const HostFr* v = reinterpret_cast<const HostFr*>(h_v);
  arena_reset(ctx);
  uint32_t *d_u, *d_v, *partial, *sums, *whi, *wlo;
  int rc;
  if ((rc = upload_fr(ctx, u, n_u, &d_u))) return rc;
  if ((rc = upload_fr(ctx, v, n_v, &d_v))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)ctx->sm_count * 4 * 3 * 8 + 64, &partial))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)(rounds_n + 1) * 3 * 8, &sums))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)first_size * 8 + 8, &whi))) return rc;
  if ((rc = arena_alloc_t(ctx, ((size_t)1 << l_in) * 8 + 8, &wlo))) return rc;
  uint32_t* A = reinterpret_cast<uint32_t*>(d_A);
  uint32_t* B = reinterpret_cast<uint32_t*>(d_B);
  std::vector<RoundInfo> rounds;
  uint64_t in_size = size, out_size = size / 2;
  uint64_t wlo_len = 0;  // inner table currently held in wlo
  for (uint32_t i = 0; i < rounds_n; i++) {
    const uint32_t* dv = d_v + (size_t)(v_end - i - 1) * 8;
    if (in_size > second_size) {
      // coefficients viewed as [out_size / N][N]: outer variables start at u[u_end - log2(first_size)],
      // inner ones at u[u_end - log2(size)]
      const uint32_t outer = (uint32_t)(out_size / second_size);
      if (wlo_len != second_size) {
        eq_weights_async(ctx, d_u + (size_t)(u_end - rounds_n) * 8, l_in, second_size, wlo);
        wlo_len = second_size;
      }
      PairWeights pw{whi, wlo, second_size};
      if (outer > 1) {
        eq_weights_async(ctx, d_u + (size_t)(u_end - l_first) * 8, log2ceil(outer), outer, whi);
        launch_round_two<true, true>(ctx, A, B, in_size, out_size, dv, pw, partial, sums + (size_t)i * 3 * 8);
      } else {
        launch_round_two<false, true>(ctx, A, B, in_size, out_size, dv, pw, partial, sums + (size_t)i * 3 * 8);
      }
    } else {
      eq_weights_async(ctx, d_u + (size_t)(u_end - rounds_n) * 8, log2ceil(out_size), (uint32_t)out_size, wlo);
      wlo_len = out_size;
      PairWeights pw{nullptr, wlo, (uint32_t)std::max<uint64_t>(out_size, 1)};
      launch_round_two<false, true>(ctx, A, B, in_size, out_size, dv, pw, partial, sums + (size_t)i * 3 * 8);
    }
    rounds.push_back({true, u[u_end - i - 1], v[v_end - i - 1]});
    in_size = out_size;
    out_size = (out_size == second_size) ? (uint64_t(1) << (log2ceil(out_size) - 1)) : out_size / 2;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  std::vector<HostFr> transcript;
  rc = finish_two(ctx, rounds, sums, A, B, reinterpret_cast<HostFr*>(h_claim), reinterpret_cast<HostFr*>(h_out_claims),
                  &transcript, "prove_eleMul");
  if (n_rounds) *n_rounds = (uint32_t)(transcript.size() / 4);
  if (h_transcript) {
    size_t n = std::min<size_t>(transcript.size(), (size_t)transcript_capacity * 4);
    memcpy(h_transcript, transcript.data(), n * 32);
  }
  return rc;
}

// combine_claims (src/prove.cu:243-301): reduces k claims X~(u_j) = c_j to one claim X~(v).
// h_us holds the k challenge vectors back to back (k * n_vars elements).  X is consumed.
extern "C" int grape_combine_claims(grape_ctx* ctx, void* d_X, uint64_t size, const void* h_claims, uint32_t k,
                                    const void* h_us, const void* h_v, uint32_t n_vars, void* h_result,
                                    void* h_transcript, uint32_t transcript_capacity, uint32_t* n_rounds) {
  if (ctx) grape::make_device_current(ctx);
  if (!ctx || !d_X || !h_claims || !h_us || !h_v || !h_result) return fail(ctx, GRAPE_ERR_INVALID, "null argument");
  if (k == 0 || k > MAX_CLAIMS) return fail(ctx, GRAPE_ERR_LIMIT, "combine_claims: between 1 and 4 claims are supported");
  if (size == 0 || (uint64_t(1) << n_vars) != size)
    return fail(ctx, GRAPE_ERR_INVALID, "combine_claims: size must equal 2^n_vars");
  const HostFr* claims = reinterpret_cast<const HostFr*>(h_claims);
  const HostFr* us = reinterpret_cast<const HostFr*>(h_us);
  const HostFr* v = reinterpret_cast<const HostFr*>(h_v);
  arena_reset(ctx);
  uint32_t *d_us, *d_v, *partial, *sums;
  int rc;
  if ((rc = upload_fr(ctx, us, (size_t)k * n_vars, &d_us))) return rc;
  if ((rc = upload_fr(ctx, v, n_vars, &d_v))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)ctx->sm_count * 4 * 2 * MAX_CLAIMS * 8 + 64, &partial))) return rc;
  if ((rc = arena_alloc_t(ctx, (size_t)(n_vars + 1) * 2 * MAX_CLAIMS * 8, &sums))) return rc;
  // weights of round i cover variables 0 .. n_vars-i-2, split into a low and a high table
  const uint32_t max_rem = n_vars ? n_vars - 1 : 0;
  const uint32_t lo_cap = (max_rem + 1) / 2, hi_cap = max_rem - lo_cap;
  ClaimWeights cw;
  for (uint32_t j = 0; j < MAX_CLAIMS; j++) {
    uint32_t *a = nullptr, *b = nullptr;
    if (j < k) {
      if ((rc = arena_alloc_t(ctx, ((size_t)1 << hi_cap) * 8 + 8, &a))) return rc;
      if ((rc = arena_alloc_t(ctx, ((size_t)1 << lo_cap) * 8 + 8, &b))) return rc;
    }
    cw.whi[j] = a;
    cw.wlo[j] = b;
  }
  uint32_t* X = reinterpret_cast<uint32_t*>(d_X);
  uint64_t out_size = size / 2;
  for (uint32_t i = 0; i < n_vars; i++) {
    const uint32_t rem = n_vars - i - 1;           // variables of the weights this round
    const uint32_t lo_bits = std::min(rem, lo_cap);
    const uint32_t hi_bits = rem - lo_bits;
    cw.lo_bits = lo_bits;
    for (uint32_t j = 0; j < k; j++) {
      const uint32_t* uj = d_us + (size_t)j * n_vars * 8;
      eq_weights_async(ctx, uj, lo_bits, 1u << lo_bits, const_cast<uint32_t*>(cw.wlo[j]));
      eq_weights_async(ctx, uj + (size_t)lo_bits * 8, hi_bits, 1u << hi_bits, const_cast<uint32_t*>(cw.whi[j]));
    }
    const uint32_t blocks = round_blocks(ctx, out_size);
    const uint32_t* dv = d_v + (size_t)(n_vars - i - 1) * 8;
    uint32_t* slot = sums + (size_t)i * 2 * MAX_CLAIMS * 8;
    switch (k) {
      case 1: k_round_one<1><<<blocks, RT, 0, ctx->stream>>>(X, out_size, dv, cw, partial);
              k_reduce_partials<2><<<1, RT, 0, ctx->stream>>>(partial, blocks, slot); break;
      case 2: k_round_one<2><<<blocks, RT, 0, ctx->stream>>>(X, out_size, dv, cw, partial);
              k_reduce_partials<4><<<1, RT, 0, ctx->stream>>>(partial, blocks, slot); break;
      case 3: k_round_one<3><<<blocks, RT, 0, ctx->stream>>>(X, out_size, dv, cw, partial);
              k_reduce_partials<6><<<1, RT, 0, ctx->stream>>>(partial, blocks, slot); break;
      default: k_round_one<4><<<blocks, RT, 0, ctx->stream>>>(X, out_size, dv, cw, partial);
               k_reduce_partials<8><<<1, RT, 0, ctx->stream>>>(partial, blocks, slot); break;
    }
    ctx->launches += 2;
    out_size /= 2;
  }
  GRAPE_CUDA_TRY(ctx, cudaGetLastError());
  std::vector<HostFr> hs((size_t)n_vars * 2 * MAX_CLAIMS + 1);
  if (n_vars) GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(hs.data(), sums, (size_t)n_vars * 2 * MAX_CLAIMS * 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaMemcpyAsync(&hs[(size_t)n_vars * 2 * MAX_CLAIMS], X, 32, cudaMemcpyDeviceToHost, ctx->stream));
  GRAPE_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  HostFr claim = fr_zero();
  for (uint32_t j = 0; j < k; j++) claim = fr_add(claim, claims[j]);
  std::vector<HostFr> E(k, fr_one());
  std::vector<HostFr> transcript;
  for (uint32_t i = 0; i < n_vars; i++) {
    const HostFr v_now = v[n_vars - i - 1];
    Poly p;
    p.n = 3;
    p.c[0] = p.c[1] = p.c[2] = fr_zero();
    for (uint32_t j = 0; j < k; j++) {
      const HostFr now_u = us[(size_t)j * n_vars + (n_vars - i - 1)];
      HostFr q[3] = {hs[(size_t)i * 2 * MAX_CLAIMS + 2 * j], hs[(size_t)i * 2 * MAX_CLAIMS + 2 * j + 1], fr_zero()};
      Poly pj = poly_mul_eq(q, now_u, E[j]);
      for (int t = 0; t < 3; t++) p.c[t] = fr_add(p.c[t], pj.c[t]);
      E[j] = fr_mul(E[j], fr_eq2(now_u, v_now));
    }
    emit(&transcript, p);
    if (poly_at01(p) != claim)
      return fail(ctx, GRAPE_ERR_CHECK, "combine_claims: claim != p(0) + p(1) in round " + std::to_string(i));
    claim = poly_eval(p, v_now);
  }
  HostFr ret = hs[(size_t)n_vars * 2 * MAX_CLAIMS];
  HostFr total = fr_zero();
  for (uint32_t j = 0; j < k; j++) total = fr_add(total, fr_mul(E[j], ret));
  if (total != claim) return fail(ctx, GRAPE_ERR_CHECK, "combine_claims: final identity failed");
  *reinterpret_cast<HostFr*>(h_result) = ret;
  if (n_rounds) *n_rounds = n_vars;
  if (h_transcript) {
    size_t n = std::min<size_t>(transcript.size(), (size_t)transcript_capacity * 4);
    memcpy(h_transcript, transcript.data(), n * 32);
  }
  return GRAPE_OK;
}
