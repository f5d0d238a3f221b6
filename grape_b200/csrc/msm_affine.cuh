// Commitment accumulation with AFFINE accumulators and shared inversions (included by msm.cu).
//
// The XYZZ kernel pays 8 multiplications and 2 squarings for every (digit, generator) pair.  In affine
// coordinates the same addition is one division, one squaring and two multiplications,
//     lambda = (y2 - y1) / (x2 - x1),   x3 = lambda^2 - x1 - x2,   y3 = lambda (x1 - x3) - y1,
// and B independent divisions share ONE inversion (Montgomery's trick: prefix products going up, one
// inversion, two multiplications per element coming back down): 5 multiplications and 1 squaring per
// addition plus 1/B of an inversion (batched division steps, mostly on the plain integer pipe, so it
// partly overlaps the other warps' multiplications: measured at 12 % of the kernel for B = 56).
//
// Independence comes from ROWS: all rows of a commitment share the generators, so a lane takes the same
// generator for B different (row, window group) slots and adds one table point to each of its B
// accumulators per step.  B accumulators of 64 bytes and B prefix products do not fit in registers or
// shared memory; they live in a scratch region of device memory, laid out so that the 32 lanes of a warp
// touch consecutive 16-byte words, and every word is read once after it was written (about 320 bytes of
// L2 / device-memory traffic per addition, table gathers included).
//
//   unit            = B consecutive slots x one chunk of generators, one warp; the lanes walk the chunk
//                     with stride 32 as in the XYZZ kernel
//   per step        = pass 1 over the slots: delta_s = x2 - x1, prefix product (saved), then one
//                     inversion, then pass 2 downwards: 1/delta_s, the addition, the new accumulator
//   special cases   = zero digit / table entry at infinity (skip), accumulator at infinity (copy),
//                     equal points (tangent: delta = 2 y, numerator 3 x^2), opposite points (back to
//                     infinity); decided from the same inputs in both passes
//   end of a unit   = lane l gathers the 32 lane sums of slots l, l + 32 with mixed XYZZ additions and
//                     writes the partial sum where the XYZZ kernel would: the finalize kernels are shared
//
// The scheme needs many rows: a warp holds 32 x B accumulators, each of which has to absorb a few dozen
// points before the closing gather stops mattering.  The host picks this kernel only then.
#pragma once

namespace grape {

constexpr int AFF_THREADS = 128;
constexpr int AFF_BLOCKS = 3;      // blocks per SM the kernel is compiled for (168 registers a thread)
constexpr uint32_t AFF_MAX_B = 64;  // slots per lane: one 64-bit mask marks the accumulators at infinity

template <class F>
struct AffineArgs {
  const void* scalars;
  TableViewT<F> tab;
  uint32_t wd, total_windows, groups;
  uint32_t n_chunks, chunk_len;
  uint64_t n_slots, n_units;
  uint32_t B;
  XyzzT<F>* partials;
  uint32_t* status;
  uint32_t inner, inner_pad;
  uint64_t n_scalars;
  uint4* scratch;  // per warp of the grid: B records of (x, y, prefix) x 32 lanes
};

template <class C, bool FR>
__global__ void __launch_bounds__(AFF_THREADS, AFF_BLOCKS) commit_accumulate_affine_kernel(
    const AffineArgs<typename C::F> a) {
  using F = typename C::F;
  using Affine = AffineT<F>;
  using Xyzz = XyzzT<F>;
  constexpr int PF = F::BYTES / 16;  // 16-byte pieces per coordinate
  constexpr int REC = 3 * PF;        // scratch record of a slot: x | y | prefix product
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warp_global = (uint64_t)blockIdx.x * (AFF_THREADS / 32) + (threadIdx.x >> 5);
  const uint64_t n_warps = (uint64_t)gridDim.x * (AFF_THREADS / 32);
  uint4* const mine = a.scratch + warp_global * ((uint64_t)a.B * REC * 32);
  // piece k of field `which` (x, y, prefix) of slot s: the 32 lanes on consecutive 16-byte words
  auto ld_lane = [&](uint32_t s, int which, uint32_t l) {
    F r;
    uint4* d = reinterpret_cast<uint4*>(r.v);
#pragma unroll
    for (int k = 0; k < PF; k++) d[k] = __ldcg(mine + ((uint64_t)(s * REC + which * PF + k) * 32 + l));
    return r;
  };
  auto ld = [&](uint32_t s, int which) { return ld_lane(s, which, lane); };
  auto st = [&](uint32_t s, int which, const F& v) {
    const uint4* src = reinterpret_cast<const uint4*>(v.v);
#pragma unroll
    for (int k = 0; k < PF; k++) __stcg(mine + ((uint64_t)(s * REC + which * PF + k) * 32 + lane), src[k]);
  };

  const TableViewT<F>& tab = a.tab;
  const uint32_t c = tab.window_bits;
  const uint32_t mask = (1u << c) - 1u;
  const uint32_t half = tab.half;
  const uint32_t tw = tab.n_windows;
  const uint32_t groups = a.groups;
  const uint32_t wd = a.wd;
  const uint32_t wd_walk = (FR && a.inner) ? wd / a.inner_pad * a.inner : wd;
  uint32_t bias32 = 0;
  if (!FR) {
    for (uint32_t w = 0; w + 1 < a.total_windows; w++) bias32 |= half << (c * w);
  }

#pragma unroll 1
  for (uint64_t unit = warp_global; unit < a.n_units; unit += n_warps) {
    const uint32_t chunk = (uint32_t)(unit % a.n_chunks);
    const uint64_t slot0 = unit / a.n_chunks * a.B;
    const uint32_t ns = (uint32_t)min((uint64_t)a.B, a.n_slots - slot0);
    const uint64_t row0 = slot0 / groups;
    const uint32_t g0 = (uint32_t)(slot0 % groups);
    const uint32_t i_begin = chunk * a.chunk_len;
    const uint32_t i_end = min(wd_walk, i_begin + a.chunk_len);
    uint64_t inf = ~0ull;  // bit s: accumulator s is the point at infinity

#pragma unroll 1
    for (uint32_t j = i_begin + lane; j < i_end; j += 32) {
      uint32_t i = j;
      if (FR && a.inner) {
        const uint32_t q = j / a.inner;
        i = q * a.inner_pad + (j - q * a.inner);
      }
#pragma unroll 1
      for (uint32_t ww = 0; ww < tw; ww++) {
        // What slot (row, g) adds in this step: 0 = nothing, else the digit's magnitude | its sign << 31.
        auto digit_code = [&](uint64_t row, uint32_t g, bool report) -> uint32_t {
          const uint32_t w = g * tw + ww;
          if (w >= a.total_windows) return 0u;
          const uint64_t idx = row * wd + i;
          int32_t d;
          bool flip;
          if (FR) {
            d = __ldg(reinterpret_cast<const int16_t*>(a.scalars) + (uint64_t)w * a.n_scalars + idx);
            flip = d < 0;
          } else {
            DigitI32 dg;
            dg.load(reinterpret_cast<const int32_t*>(a.scalars) + idx, bias32);
            d = i32_digit(dg.vb, w, c, mask, half, a.total_windows);
            flip = (d < 0) != dg.neg;
          }
          if (d == 0) return 0u;
          const uint32_t mag = d < 0 ? (uint32_t)(-d) : (uint32_t)d;
          if (!FR && mag > half) {  // scalar larger than the declared bound: report, never read out of range
            if (report) atomicOr(a.status, STATUS_DIGIT_RANGE);
            return 0u;
          }
          return mag | (flip ? 0x80000000u : 0u);
        };
        auto entry_of = [&](uint32_t code) {
          return reinterpret_cast<const char*>(tab.entry(ww, code & 0x7fffffffu, i));
        };
        auto load_y2 = [&](uint32_t code) {
          F y = F::load_nc(entry_of(code) + F::BYTES);
          return (code >> 31) ? fe_neg(y) : y;
        };
        // Both passes run as a software pipeline: the digit of slot s +- 2 and the operands of slot
        // s +- 1 (table record, accumulator, prefix product) are requested before slot s is computed, so
        // that a slot's arithmetic covers the next slot's memory latency.  The special cases (table entry
        // or accumulator at infinity, equal or opposite points) are decided from the same inputs in
        // both passes.

        // pass 1, upwards: prefix products of the denominators delta_s = x2 - x1
        F run = F::one();
        bool any = false;
        {
          uint64_t crow = row0;  // cursor of the digit loads
          uint32_t cg = g0;
          auto advance = [&]() {
            if (++cg == groups) {
              cg = 0;
              crow++;
            }
          };
          uint32_t code_a = digit_code(crow, cg, true), code_b = 0;
          advance();
          if (ns > 1) {
            code_b = digit_code(crow, cg, true);
            advance();
          }
          F nx2 = F::zero(), nx1;
          if (code_a) nx2 = F::load_nc(entry_of(code_a));
          nx1 = ld(0, 0);
#pragma unroll 1
          for (uint32_t s = 0; s < ns; s++) {
            const uint32_t code = code_a;
            const F x2 = nx2, x1 = nx1;
            code_a = code_b;
            code_b = 0;
            if (s + 2 < ns) {
              code_b = digit_code(crow, cg, true);
              advance();
            }
            if (s + 1 < ns) {
              if (code_a) nx2 = F::load_nc(entry_of(code_a));
              nx1 = ld(s + 1, 0);
            }
            if (code == 0) continue;
            if (x2.is_zero() && load_y2(code).is_zero()) continue;  // table entry at infinity
            if ((inf >> s) & 1ull) continue;                         // copy: no division
            F delta = fe_sub(x2, x1);
            if (delta.is_zero()) {
              const F y2 = load_y2(code), y1 = ld(s, 1);
              if (y1 == y2 && !y1.is_zero()) delta = fe_dbl(y1);  // tangent
              else continue;                                       // opposite points
            }
            st(s, 2, run);
            run = fe_lmul(run, delta);
            any = true;
          }
        }
        F inv = any ? fe_inv(fe_canon(run)) : F::one();
        // pass 2, downwards: 1 / delta_s = inv * prefix_s, then inv *= delta_s
        {
          const uint64_t last = slot0 + ns - 1;
          uint64_t crow = last / groups;
          uint32_t cg = (uint32_t)(last % groups);
          auto retreat = [&]() {
            if (cg == 0) {
              cg = groups - 1;
              crow--;
            } else {
              cg--;
            }
          };
          uint32_t code_a = digit_code(crow, cg, false), code_b = 0;
          retreat();
          if (ns > 1) {
            code_b = digit_code(crow, cg, false);
            retreat();
          }
          F nx2 = F::zero(), ny2 = F::zero(), nx1, ny1, npre;
          if (code_a) {
            const char* e = entry_of(code_a);
            nx2 = F::load_nc(e);
            ny2 = F::load_nc(e + F::BYTES);
          }
          nx1 = ld(ns - 1, 0);
          ny1 = ld(ns - 1, 1);
          npre = ld(ns - 1, 2);
#pragma unroll 1
          for (uint32_t s = ns; s-- > 0;) {
            const uint32_t code = code_a;
            const F x2 = nx2, x1 = nx1, y1 = ny1, pre = npre;
            F y2 = ny2;
            code_a = code_b;
            code_b = 0;
            if (s >= 2) {
              code_b = digit_code(crow, cg, false);
              retreat();
            }
            if (s >= 1) {
              if (code_a) {
                const char* e = entry_of(code_a);
                nx2 = F::load_nc(e);
                ny2 = F::load_nc(e + F::BYTES);
              }
              nx1 = ld(s - 1, 0);
              ny1 = ld(s - 1, 1);
              npre = ld(s - 1, 2);
            }
            if (code == 0) continue;
            if (code >> 31) y2 = fe_neg(y2);
            if (x2.is_zero() && y2.is_zero()) continue;
            if ((inf >> s) & 1ull) {
              st(s, 0, x2);
              st(s, 1, y2);
              inf &= ~(1ull << s);
              continue;
            }
            F delta = fe_sub(x2, x1);
            F num;
            if (delta.is_zero()) {
              if (y1 == y2 && !y1.is_zero()) {
                delta = fe_dbl(y1);
                const F xx = fe_lsqr(x1);
                num = fe_ladd(fe_ladd(xx, xx), xx);
              } else {
                inf |= 1ull << s;
                continue;
              }
            } else {
              num = fe_sub(y2, y1);
            }
            const F dinv = fe_lmul(inv, pre);
            inv = fe_lmul(inv, delta);
            const F lam = fe_lmul(num, dinv);
            const F x3 = fe_lsub(fe_lsub(fe_lsqr(lam), x1), x2);  // a tangent has x2 == x1
            const F y3 = fe_lsub(fe_lmul(lam, fe_lsub(x1, x3)), y1);
            st(s, 0, fe_canon(x3));
            st(s, 1, fe_canon(y3));
          }
        }
      }
    }

    // the lane sums of every slot become one partial sum: (0, 0) marks a lane sum at infinity
#pragma unroll 1
    for (uint32_t s = 0; s < ns; s++) {
      if ((inf >> s) & 1ull) {
        st(s, 0, F::zero());
        st(s, 1, F::zero());
      }
    }
    __syncwarp();
#pragma unroll 1
    for (uint32_t s = lane; s < ns; s += 32) {
      Xyzz acc = Xyzz::inf();
#pragma unroll 1
      for (uint32_t l = 0; l < 32; l++) {
        Affine q;
        q.x = ld_lane(s, 0, l);
        q.y = ld_lane(s, 1, l);
        xyzz_madd_lazy(acc, q);
      }
      xyzz_canon(acc).store(a.partials + (slot0 + s) * a.n_chunks + chunk);
    }
    __syncwarp();  // the next unit overwrites the records
  }
}

// How the affine kernel would cut `slots` accumulation streams of `walk` generators (times the table's
// windows per group) into units, and what that costs next to the XYZZ kernel; both in multiplications per
// multiplier pipe.  use == false when the XYZZ kernel is expected to win (few rows, short rows).
struct AffinePlan {
  bool use = false;
  uint32_t B = 0, n_chunks = 1, chunk_len = 0;
  uint64_t units = 0, grid_warps = 0;
};

// Multiplication-equivalents, measured on the 8-limb field: a lazy product 1, a lazy square 0.79, hence
// an affine addition 5.8 and a mixed XYZZ addition 9.6; an inversion as seen by a warp whose
// neighbours keep the multiplier busy meanwhile.
constexpr double AFF_COST_ADD = 5.8, AFF_COST_MADD = 9.6, AFF_COST_INV = 30.0;
// This kernel keeps the multiplier pipe 64 % busy where the XYZZ kernel reaches 87 % (twelve warps per SM
// against sixteen, operands from device memory): measured 28.8 ms where the counts alone say 22.
constexpr double AFF_PIPE_PENALTY = 1.3;

static AffinePlan plan_affine(const grape_ctx* ctx, uint64_t slots, uint32_t walk, uint32_t tw, bool force,
                              int force_b, int force_chunks) {
  AffinePlan best;
  if (slots == 0 || walk == 0) return best;
  const uint64_t R = (uint64_t)ctx->sm_count * AFF_BLOCKS * (AFF_THREADS / 32);  // warps resident at once
  // the XYZZ kernel keeps the multiplier pipe about as busy with 16 warps as this kernel with 12, so
  // both costs are counted per pipe: work of all lanes / number of pipes
  const double pipes = (double)ctx->sm_count * 4 * 32;
  const double cost_xyzz = (double)slots * walk * tw * AFF_COST_MADD / pipes;
  double best_cost = force ? 1e300 : cost_xyzz * 0.92;  // unforced: switch only for a clear gain
  for (uint32_t B = force_b ? (uint32_t)force_b : AFF_MAX_B; B >= (force_b ? 1u : 8u); B -= 8) {
    if (!force_b && B > slots && B > 8) continue;
    const uint64_t blocks = (slots + B - 1) / B;
    for (uint32_t waves = 1; waves <= 4; waves++) {
      uint64_t c = force_chunks ? (uint64_t)force_chunks : waves * R / blocks;
      if (c == 0) c = 1;
      const uint32_t max_c = (walk + 31) / 32;
      if (c > max_c) c = max_c;
      uint32_t chunk_len = (uint32_t)((walk + c - 1) / c);
      chunk_len = (chunk_len + 31) / 32 * 32;
      c = (walk + chunk_len - 1) / chunk_len;
      const uint64_t units = blocks * c;
      const uint64_t rounds = (units + R - 1) / R;  // units per warp of the grid
      const double steps = (double)(chunk_len / 32) * tw;
      const double unit_cost = steps * (B * AFF_COST_ADD + AFF_COST_INV) + (double)((B + 31) / 32) * 32 * AFF_COST_MADD;
      // a round keeps min(units, R) warps busy: R warps share the pipes
      const double cost = AFF_PIPE_PENALTY * (double)rounds * unit_cost * (double)R * 32 / pipes;
      if (cost < best_cost) {
        best_cost = cost;
        best.use = true;
        best.B = B;
        best.n_chunks = (uint32_t)c;
        best.chunk_len = chunk_len;
        best.units = units;
        best.grid_warps = units < R ? units : R;
      }
      if (force_chunks) break;
    }
    if (force_b) break;
  }
  return best;
}

}  // namespace grape
