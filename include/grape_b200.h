/*
 * grape_b200 -- C ABI of the B200 (sm_100a) proving hot path.
 *
 * This is the boundary a caller written against the reference's static library binds instead of
 * the reference's CUDA sources.  Every entry point names the reference interface it replaces
 * (path:line inside the reference project).  All functions return a GRAPE_* status, never throw,
 * never trap the device; grape_ctx_error() returns the text of the last failure on a context.
 *
 * Data formats (identical to the reference's device records):
 *   Fr element    32 B  eight little-endian 32-bit limbs, Montgomery form (value * 2^256 mod r)
 *   affine point  64 B  X|Y over Fp, Montgomery form, all-zero = point at infinity
 *   Jacobian      96 B  X|Y|Z; outputs are always normalised to Z = 1 (or X=Y=1, Z=0 for
 *                       infinity) so that equal group elements have equal bytes
 * Pointers whose name starts with d_ are device pointers on the context's GPU, h_ are host.
 * Calls on one context are issued on that context's stream and are asynchronous unless stated.
 */
#ifndef GRAPE_B200_H
#define GRAPE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GRAPE_OK 0
#define GRAPE_ERR_INVALID 1 /* bad argument / shape (reference: std::runtime_error) */
#define GRAPE_ERR_CUDA 2    /* CUDA runtime failure, text in grape_ctx_error */
#define GRAPE_ERR_CHECK 3   /* a prover-side round check p(0)+p(1)==claim failed */
#define GRAPE_ERR_NOMEM 4
#define GRAPE_ERR_LIMIT 5 /* size beyond a documented fixed limit */

#define GRAPE_FR_BYTES 32
#define GRAPE_AFFINE_BYTES 64
#define GRAPE_JACOBIAN_BYTES 96
#define GRAPE_BLS12_381_AFFINE_BYTES 96
#define GRAPE_BLS12_381_JACOBIAN_BYTES 144
#define GRAPE_CURVE_BN254 0u
#define GRAPE_CURVE_BLS12_381 1u
#define GRAPE_COM_SCALE 16 /* reference: Hyrax::com_scale, src/Hyrax.cu:229 */

typedef struct grape_ctx grape_ctx;
typedef struct grape_table grape_table;
typedef struct grape_lookup grape_lookup;

/* ---- context ------------------------------------------------------------------------------ */
/* One context = one GPU + one stream + a grow-only scratch arena + the prover's random stream.
 * The reference has no such object (single device, default stream, src/Hyrax.cu:312-333 allocates
 * and frees scratch in every call).  Every call that takes a context makes the context's GPU the
 * calling thread's current CUDA device and leaves it so; one host thread at a time per context. */
int grape_ctx_create(int device, grape_ctx** out);
int grape_ctx_destroy(grape_ctx* ctx);
const char* grape_ctx_error(const grape_ctx* ctx);
int grape_ctx_sync(grape_ctx* ctx);
void* grape_ctx_stream(grape_ctx* ctx); /* cudaStream_t */
int grape_version(void);

/* The stream that replaces libff's Fr::random_element() inside the provers (reference draws:
 * src/tlookup.cu:247,293,351,403; src/Hyrax.cu:253-256: the lookups' alpha, r and u, the blinding
 * vector of every opening).  A new context draws from ChaCha20 under a 256-bit key taken from the
 * operating system (grape_ctx_create fails without one), 512 bits per element reduced mod r.
 * grape_rng_seed switches the context to a REPLAYABLE SplitMix64 stream with 64 bits of state, the
 * one the oracle and the reference stand-in use, so that tests can compare proofs bit for bit.
 * Security: with a seeded stream the blinders are predictable and z = c*x + d reveals x; never
 * seed a context whose proofs must hide their witness. */
int grape_rng_seed(grape_ctx* ctx, uint64_t seed);
/* Draws n Fr elements (Montgomery form) from the context's stream into host memory. */
int grape_rng_fr(grape_ctx* ctx, void* h_out, uint64_t n);

/* ---- raw device memory (so that FFI callers need not bind the CUDA runtime) ---------------- */
int grape_dev_alloc(grape_ctx* ctx, size_t bytes, void** d_out);
int grape_dev_free(grape_ctx* ctx, void* d_ptr);
int grape_h2d(grape_ctx* ctx, void* d_dst, const void* h_src, size_t bytes); /* async */
/* The same copy on a second stream, overlapping the kernels queued on the context's main stream
 * (h_src page-locked).  It starts after the work queued so far; grape_prefetch_wait(ticket) makes
 * the main stream wait for that copy and releases the ticket.  Lets a driver load the tensors of
 * later steps while the current one is proven (the reference's driver loads synchronously,
 * src/ioutils.cu:105-124). */
int grape_h2d_prefetch(grape_ctx* ctx, void* d_dst, const void* h_src, size_t bytes, uint32_t* ticket);
int grape_prefetch_wait(grape_ctx* ctx, uint32_t ticket);
int grape_d2h(grape_ctx* ctx, void* h_dst, const void* d_src, size_t bytes); /* synchronises */
int grape_d2d(grape_ctx* ctx, void* d_dst, const void* d_src, size_t bytes);
int grape_dev_zero(grape_ctx* ctx, void* d_dst, size_t bytes);

/* ---- generator table ---------------------------------------------------------------------- */
/* Fixed-base table  T[w][d-1][i] = (2^(window_bits*w) * d) * G_i  for d in 1..2^(window_bits-1),
 * w < n_windows, affine.  Replaces precompute_generators / naive_msm
 * (src/ec_operation.cu:15-49), whose table is w*G_i for w < 256.  window_bits is 5..16: wider
 * windows mean fewer additions per scalar and a table of 2^(window_bits-1) * n_gens * 64 bytes per window.
 * d_gens_jacobian: n_gens Jacobian records (the reference's cpu_points layout). */
int grape_table_create(grape_ctx* ctx, const void* d_gens_jacobian, uint32_t n_gens,
                       uint32_t window_bits, uint32_t n_windows, grape_table** out);
/* Wraps a table laid out like the reference's points.bin: 256 rows of n_gens affine points,
 * row w = w*G_i (src/ec_operation.cu:24).  Borrows d_points (no copy). */
int grape_table_from_reference(grape_ctx* ctx, const void* d_points, uint32_t n_gens,
                               grape_table** out);
/* The same table over BLS12-381 G1 (y^2 = x^3 + 4; Fp on twelve 32-bit limbs with Montgomery radix
 * 2^384, Fr on eight with radix 2^256 -- the constants of include/field/bls12-381.cuh:7-46, which the
 * reference defines but compiles nothing against, so there is no reference call site).  Records are
 * 3/2 the BN254 sizes: generators and commitments are 144-byte Jacobian records (X|Y|Z, 48 B each),
 * table entries 96-byte affine records.  grape_commit_i32, grape_commit_fr and
 * grape_commit_i32_host accept such a table and then read BLS12-381 Fr scalars / write 144-byte
 * records; the opening and lookup entry points reject it. */
int grape_bls12_381_table_create(grape_ctx* ctx, const void* d_gens_jacobian, uint32_t n_gens,
                                 uint32_t window_bits, uint32_t n_windows, grape_table** out);
/* GRAPE_CURVE_BN254 or GRAPE_CURVE_BLS12_381. */
uint32_t grape_table_curve(const grape_table* t);
int grape_table_destroy(grape_table* t);
uint64_t grape_table_bytes(const grape_table* t);
const void* grape_table_data(const grape_table* t);

/* ---- Hyrax row commitments ---------------------------------------------------------------- */
/* C_r = sum_{i<wd} s[r*wd+i] * G_i for the rows of an int32 tensor.
 * Replaces Hyrax::commit(int*, size, N) (src/Hyrax.cu:312-333, kernels :46-87) with wd = N*16.
 * max_bits: bound on the magnitude of the scalars, |s| <= 2^(max_bits-1) (32 = any int32,
 * 16 = int16-range data); it only trims windows that are known to be zero.
 * d_out: size/wd Jacobian records. */
int grape_commit_i32(grape_ctx* ctx, const grape_table* t, const int32_t* d_scalars, uint64_t size,
                     uint32_t wd, uint32_t max_bits, void* d_out);
/* Same for Fr scalars (Montgomery form, not modified).  Replaces Hyrax::commit(FrTensor&, size, N)
 * (src/Hyrax.cu:335-359, kernels :128-167) and single_commit (src/Hyrax.cu:176-185) for one row. */
int grape_commit_fr(grape_ctx* ctx, const grape_table* t, const void* d_scalars, uint64_t size,
                    uint32_t wd, void* d_out);
/* Host-buffer form of grape_commit_i32: brings the scalars in, commits, copies the Jacobian
 * records out and synchronises (reference flow: load_data + commit + savebin, test/commit.cu:60-72).
 * Page-locked scalars (cudaMallocHost / cudaHostAlloc / grape_host_alloc_pinned) are read by the kernel
 * in place across PCIe; pageable ones are copied in row slices that overlap the commitment of the
 * slice before.  The buffer must stay valid until the call returns (it synchronises). */
int grape_commit_i32_host(grape_ctx* ctx, const grape_table* t, const int32_t* h_scalars,
                          uint64_t size, uint32_t wd, uint32_t max_bits, void* h_out);

/* ---- field tensors over Fr ---------------------------------------------------------------- */
/* Device arrays of 32-byte Montgomery residues; n counts elements.  These replace the FrTensor
 * kernels of src/fr-tensor.cu; outputs may alias inputs unless stated. */
int grape_fr_from_i32(grape_ctx* ctx, const int32_t* d_in, void* d_out, uint64_t n);   /* int_to_fr :30-39 */
int grape_fr_from_u32(grape_ctx* ctx, const uint32_t* d_in, void* d_out, uint64_t n);  /* uint_to_fr :41-46 */
int grape_fr_to_mont(grape_ctx* ctx, void* d_t, uint64_t n);                           /* to_kernel :116-120 */
int grape_fr_from_mont(grape_ctx* ctx, void* d_t, uint64_t n);                         /* from_kernel :110-114 */
int grape_fr_add(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n); /* :74-79 */
int grape_fr_sub(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n); /* :81-86 */
int grape_fr_mul(grape_ctx* ctx, const void* d_a, const void* d_b, void* d_out, uint64_t n); /* :96-101 */
/* out = a * s / out = a + s with s one Fr element in device memory (Fr_broadcast_mul/add :88-108) */
int grape_fr_scale(grape_ctx* ctx, const void* d_a, const void* d_scalar, void* d_out, uint64_t n);
int grape_fr_add_scalar(grape_ctx* ctx, const void* d_a, const void* d_scalar, void* d_out, uint64_t n);
/* out = a * s + b  (z = c*x + d of Hyrax::open, src/Hyrax.cu:281-284) */
int grape_fr_axpy(grape_ctx* ctx, const void* d_a, const void* d_scalar, const void* d_b, void* d_out,
                  uint64_t n);
/* out[i] = 1 / (in[i] + shift) with shift one device Fr element or NULL; zero maps to zero.
 * Replaces inverse_kernel (:122-126) and tlookup_inv_kernel (src/tlookup.cu:52-62); batched. */
int grape_fr_inverse(grape_ctx* ctx, const void* d_in, const void* d_shift, void* d_out, uint64_t n);
/* Row padding n -> pad_n over pad_size output elements (pad_int_kernel / pad_fr_kernel :18-28).
 * d_out must not alias d_in. */
int grape_pad_i32(grape_ctx* ctx, const int32_t* d_in, int32_t* d_out, uint32_t n, uint32_t pad_n,
                  uint64_t pad_size);
int grape_fr_pad(grape_ctx* ctx, const void* d_in, void* d_out, uint32_t n, uint32_t pad_n,
                 uint64_t pad_size, const void* d_pad_value);
/* d_out[0] = sum of the first n elements (FrTensor::sum(sz), :415-440). */
int grape_fr_sum(grape_ctx* ctx, const void* d_in, uint64_t n, void* d_out);
/* Every element of a row replaced by the row sum (FrTensor::sum(sz, N) / sum_by_dim_kernel :155-163). */
int grape_fr_rowsum(grape_ctx* ctx, const void* d_in, void* d_out, uint64_t rows, uint32_t dim);
/* Multilinear fold of one axis: the first ntot elements of d_t are viewed as [other][c][gap]; axis c
 * is folded with the challenges d_x[0 .. ceil(log2 c)) (variable 0 = lowest index bit, odd tails
 * paired with zero) into d_out = [other][gap].  Same values as FrTensor::partial_eval(N, x, c, id, gap)
 * (:53-72,168-188,330-344) called with x + id; d_out must not alias d_t, which is left intact. */
int grape_fr_fold(grape_ctx* ctx, const void* d_t, uint64_t ntot, const void* d_x, uint32_t c,
                  uint64_t gap, void* d_out);
/* The same fold reading an int32 tensor directly (skips the 8x larger Fr copy the reference
 * materialises first, src/fr-tensor.cu:376-381). */
int grape_fold_i32(grape_ctx* ctx, const int32_t* d_t, uint64_t ntot, const void* d_x, uint32_t c,
                   uint64_t gap, void* d_out);

/* ---- sumcheck provers ----------------------------------------------------------------------- */
/* Challenge vectors and claims are host arrays of 32-byte Fr elements (the reference's
 * std::vector<Fr> / Fr).  h_claim is read (claimed value) and overwritten with the final running
 * claim; a failed round check p(0)+p(1)==claim returns GRAPE_ERR_CHECK where the reference throws.
 * h_transcript (may be NULL) receives up to transcript_capacity round polynomials of four
 * coefficients each, lowest degree first (degree-2 rounds end with a zero); *n_rounds the count.
 * Tensor arguments are consumed (left folded), as in the reference. */

/* prove_matmul (src/prove.cu:175-210; phases :49-117).  d_A = [L][N][K], d_B = [L][M][K];
 * u = u_M | u_N | u_L, v = v_K | v_L.  h_out_claims[0..1] = A~(v_K,u_N,v_L), B~(v_K,u_M,v_L). */
int grape_prove_matmul(grape_ctx* ctx, void* d_A, void* d_B, uint32_t L, uint32_t N, uint32_t M, uint32_t K,
                       const void* h_u, uint32_t n_u, const void* h_v, uint32_t n_v, void* h_claim,
                       void* h_out_claims, void* h_transcript, uint32_t transcript_capacity,
                       uint32_t* n_rounds);

/* prove_matmul straight from the int32 tensors that the reference turns into FrTensors right before
 * the call (FrTensor(uint size, int* data), src/fr-tensor.cu:190-197; e.g. test/matmul.cu).  Same
 * outputs as grape_fr_from_i32 on both tensors followed by grape_prove_matmul; d_A and d_B are
 * left intact.  A veneer FrTensor that still holds its int32 source can bind prove_matmul here. */
int grape_prove_matmul_i32(grape_ctx* ctx, const int32_t* d_A, const int32_t* d_B, uint32_t L, uint32_t N,
                           uint32_t M, uint32_t K, const void* h_u, uint32_t n_u, const void* h_v,
                           uint32_t n_v, void* h_claim, void* h_out_claims, void* h_transcript,
                           uint32_t transcript_capacity, uint32_t* n_rounds);

/* prove_matmul split over P = 2^p provers (GPUs), one exchange in total.  No reference counterpart:
 * the reference proves on one GPU (src/prove.cu:175-210); the result and the transcript are
 * bit-identical to grape_prove_matmul on the unsharded tensors.
 *   Sharding: prover r holds the inner-dimension columns k = k'*P + r of A and B as dense
 *   [L][N][K/P] and [L][M][K/P] Fr tensors (P must divide K).  The rounds over the top
 *   log2ceil(K) - p inner variables, and the layer variables before them, never pair elements of
 *   different provers, and all challenges are inputs, so each prover runs them alone.
 *   grape_prove_matmul_partial (every prover, asynchronous on the context's stream): writes
 *   (3*local_rounds + 2) field elements to d_part (device memory): per-round partial sums, then the
 *   shard's fully folded A and B values.  h_v_local = v without its p lowest entries.
 *   The caller gathers the P d_part buffers in rank order (e.g. an NCCL all-gather) into d_gathered.
 *   grape_prove_matmul_finish: adds the partial sums mod r on the device, runs the last p rounds
 *   over the P folded values, then checks every round (GRAPE_ERR_CHECK) and returns the claims and
 *   the transcript exactly as grape_prove_matmul does. */
int grape_prove_matmul_partial(grape_ctx* ctx, void* d_A_shard, void* d_B_shard, uint32_t L, uint32_t N,
                               uint32_t M, uint32_t K_local, const void* h_u, uint32_t n_u,
                               const void* h_v_local, uint32_t n_v_local, void* d_part, uint32_t* local_rounds);
int grape_prove_matmul_finish(grape_ctx* ctx, const void* d_gathered, uint32_t P, uint32_t L, uint32_t N,
                              uint32_t M, uint32_t K, const void* h_u, uint32_t n_u, const void* h_v,
                              uint32_t n_v, void* h_claim, void* h_out_claims, void* h_transcript,
                              uint32_t transcript_capacity, uint32_t* n_rounds);
/* prove_eleMul (src/prove.cu:212-241; eleMul_sumcheck :119-172).  d_A, d_B = [L*M][N]. */
int grape_prove_elemul(grape_ctx* ctx, void* d_A, void* d_B, uint32_t L, uint32_t M, uint32_t N,
                       const void* h_u, uint32_t n_u, const void* h_v, uint32_t n_v, void* h_claim,
                       void* h_out_claims, void* h_transcript, uint32_t transcript_capacity,
                       uint32_t* n_rounds);
/* combine_claims (src/prove.cu:243-301): k <= 4 claims X~(u_j) = c_j -> h_result = X~(v).
 * h_us: the k challenge vectors back to back (k * n_vars elements); size = 2^n_vars. */
int grape_combine_claims(grape_ctx* ctx, void* d_X, uint64_t size, const void* h_claims, uint32_t k,
                         const void* h_us, const void* h_v, uint32_t n_vars, void* h_result,
                         void* h_transcript, uint32_t transcript_capacity, uint32_t* n_rounds);

/* ---- lookup argument ------------------------------------------------------------------------ */
/* tLookupRange(low, len) (src/tlookup.cu:251-263): table low .. low+2^ceil(log2 len)-1, beta = table
 * size, alpha drawn from the context's random stream. */
int grape_lookup_range_create(grape_ctx* ctx, int32_t low, uint32_t len, grape_lookup** out);
/* tLookupRangeMapping(low, len, file) (src/tlookup.cu:350-371) with the int32 table f already in
 * device memory (len a power of two); draws alpha then r. */
int grape_lookup_mapping_create(grape_ctx* ctx, int32_t low, uint32_t len, const int32_t* d_map,
                                grape_lookup** out);
int grape_lookup_destroy(grape_lookup* lk);
/* alpha, beta, r (32 bytes each, any may be NULL) and the table size. */
int grape_lookup_params(const grape_lookup* lk, void* h_alpha, void* h_beta, void* h_r, uint32_t* n);
/* What a verifier of the LAST successful prove on this object needs besides the round polynomials
 * (no counterpart in the reference, whose tLookup_phase2 returns S~(v) alone, src/tlookup.cu:195,
 * and whose only checks are the prover-side p(0)+p(1) tests, src/tlookup.cu:203,231):
 *   h_finals: five Fr elements A~(v), S~(v), B~(v_low), T~(v_low), m~(v_low), the tensors of the
 *             argument folded down to one value each (v_low = the log2(table size) low challenges);
 *   h_u:      the ceil(log2 D) elements the prover drew for u (src/tlookup.cu:293), *n_u of them.
 * Either pointer may be NULL.  GRAPE_ERR_INVALID when no proof has been produced yet. */
int grape_lookup_last_proof(const grape_lookup* lk, void* h_finals, void* h_u, uint32_t u_capacity, uint32_t* n_u);
/* Device time, in seconds, that the commitments of A and m took inside the last prove with a table
 * (what the reference adds to its commit_time argument, src/tlookup.cu:319-323); 0 without one. */
int grape_lookup_last_commit_seconds(const grape_lookup* lk, double* seconds);
/* Device tensors of the object: 0 = T, 1 = B = 1/(T+beta), 2 = m (multiplicities of the last
 * prove), 3 = mapped values. */
const void* grape_lookup_table(const grape_lookup* lk, int which);
/* How the lookup provers commit A = 1/(S+beta) (no reference counterpart; the commitment is the same
 * group element either way).  Every A_i equals the table's B[t] for the entry t that S_i hits, so a
 * commitment row with several times more elements than the table has entries is cheaper by the
 * bucket method: add up the generators per table entry first (one addition per element), then one
 * variable-base multi-scalar multiplication of those sums by B per row.
 * mode 0: never; 1 (default): when the measured cost model favours it (rows at least about seven
 * times longer than the table has entries); 2: whenever the shape allows. */
int grape_lookup_set_bucket_commit(grape_ctx* ctx, int mode);

/* Which kernel accumulates the row commitments (no reference counterpart; the commitments are the same
 * group elements either way).  With many rows the additions of different rows are independent, so they
 * can run in affine coordinates with one shared inversion per batch (6 field multiplications per
 * addition instead of 10), at the price of keeping the accumulators in device memory.  Measured on a
 * B200 it gains 10 % on 49 408 rows x 4096 generators of int16 scalars, 8 % on a whole layer proof (the
 * lookups' full-width A tensors) and loses below some tens of millions of additions.
 * mode 0: never the affine kernel; 1: when its cost model expects a clear gain; 2: always, with
 * slots_per_lane accumulators per lane (up to 64, 0 = chosen) and `chunks` chunks of generators per
 * block of rows (0 = chosen) -- for measurements.  A new context starts with mode 1 for Fr-scalar
 * commitments (grape_commit_fr, the lookup provers) and mode 0 for int32-scalar ones; this call sets
 * both, and mode -1 restores that starting state. */
int grape_commit_set_affine(grape_ctx* ctx, int mode, int slots_per_lane, int chunks);

/* tLookupRange::prove (src/tlookup.cu:288-343).  d_S: D queries; when D is not a power of two the
 * rows of length `inner` are padded to `inner_pad` (the reference hard-codes 11008 -> 16384) and
 * d_S, d_A must hold 2^ceil(log2 D) elements.  d_A receives 1/(S+beta); both are consumed.
 * table / msm_size: commit A (rows of msm_size*16) and the multiplicities as the reference does
 * (pass table = NULL to skip); d_com_A / d_com_m (may be NULL) receive those commitments.
 * h_claim = S~(v).  Draws ceil(log2 D) elements from the random stream (the reference's u). */
int grape_lookup_prove_range(grape_ctx* ctx, grape_lookup* lk, void* d_S, uint64_t D, void* d_A,
                             const void* h_v, uint32_t n_v, uint32_t inner, uint32_t inner_pad,
                             const grape_table* table, uint32_t msm_size, void* d_com_A, void* d_com_m,
                             void* h_claim, void* h_transcript, uint32_t transcript_capacity,
                             uint32_t* n_rounds);
/* tLookupRangeMapping::prove (src/tlookup.cu:398-456): pairs (S_in, S_out = f(S_in)); d_S_work
 * (2^ceil(log2 D) elements) receives S_in + r*S_out. */
int grape_lookup_prove_mapping(grape_ctx* ctx, grape_lookup* lk, const void* d_S_in, const void* d_S_out,
                               uint64_t D, void* d_S_work, void* d_A, const void* h_v, uint32_t n_v,
                               uint32_t inner, uint32_t inner_pad, const grape_table* table,
                               uint32_t msm_size, void* d_com_A, void* d_com_m, void* h_claim,
                               void* h_transcript, uint32_t transcript_capacity, uint32_t* n_rounds);

/* ---- Hyrax opening -------------------------------------------------------------------------- */
/* Hyrax::open (src/Hyrax.cu:237-305).  d_tensor = [layer_num][rows][N*16] Fr (left intact here; the
 * reference destroys it), size its element count, h_eval_point = ceil(log2 size) challenges, h_c the
 * verifier's scalar, h_G_jacobian the base point (the reference passes cpu_points[0]).  The blinding
 * vector d (16 * 2^ceil(log2 N) elements) is drawn from the context's random stream.  Outputs (host):
 * h_result = tensor~(eval_point), h_z = c*x + d (16 * 2^ceil(log2 N) elements), h_com_d = sum d_i G_i,
 * h_com_ad = <eq(eval_point), d> * G, both as normalised Jacobian records (Hyrax_proof, include/Hyrax.cuh:57-69). */
int grape_hyrax_open(grape_ctx* ctx, const grape_table* table, const void* d_tensor, uint64_t size, uint32_t N,
                     uint32_t layer_num, const void* h_eval_point, uint32_t n_e, const void* h_c,
                     const void* h_G_jacobian, void* h_result, void* h_z, void* h_com_d, void* h_com_ad);

/* ---- host-side Fr arithmetic ---------------------------------------------------------------- */
/* What the reference does with libff's Fr on the host (claim algebra, src/prove.cu:55-82,
 * test/llm.cu:98-108).  Host pointers to 32-byte Montgomery elements; outputs may alias inputs. */
void grape_hfr_add(const void* a, const void* b, void* out);
void grape_hfr_sub(const void* a, const void* b, void* out);
void grape_hfr_mul(const void* a, const void* b, void* out);
void grape_hfr_inv(const void* a, void* out);
void grape_hfr_from_i64(int64_t v, void* out);

/* ---- verifier-side group arithmetic ---------------------------------------------------------- */
/* out = sum_i s_i * P_i over n arbitrary Jacobian points and Fr scalars (device memory); d_out is one
 * normalised Jacobian record.  Replaces the libff host code of the reference's only verifier
 * (host_partial_me<G1>, Fr * G1: include/ec_operation.cuh:37-55, test/HyraxTest.cu:96-125). */
int grape_g1_lincomb(grape_ctx* ctx, const void* d_points_jacobian, const void* d_scalars, uint64_t n,
                     void* d_out);

/* ---- host-side group arithmetic for drivers (not on the proving path) ------------------------- */
/* What the reference's drivers do with libff's alt_bn128_G1 on the host: the verifier identities of
 * test/HyraxTest.cu:88-125, host_partial_me<bn128> (include/ec_operation.cuh:37-55).  All pointers are
 * HOST pointers to 96-byte Jacobian records (X|Y|Z Montgomery, Z = 0 infinity), any Z accepted;
 * scalars are 32-byte Montgomery Fr.  Thread-safe (no state). */
void grape_hg1_add(const void* h_a, const void* h_b, void* h_out);
void grape_hg1_scalar_mul(const void* h_fr, const void* h_point, void* h_out);
void grape_hg1_neg(const void* h_a, void* h_out);
void grape_hg1_normalise(const void* h_a, void* h_out); /* Z = 1, or (1, 1, 0) for infinity */
int grape_hg1_equal(const void* h_a, const void* h_b);  /* 1 when the two records are the same group element */

/* ---- allocation-free commitment ------------------------------------------------------------ */
/* No counterpart in the reference (its commit allocates and frees scratch on every call,
 * src/Hyrax.cu:312-333).  For embedders that may not allocate GPU memory when they commit --
 * a framework that owns all device memory through its own pool, a serving loop that cannot
 * afford cudaMalloc's implicit device synchronisation -- this variant of grape_commit_i32 keeps
 * its per-(row, chunk) partial sums in a fixed 8 MiB array inside the library image instead of
 * the context's arena.  It takes no context: d_table / n_gens / window_bits / n_windows describe
 * a BN254 table as grape_table_create lays it out (grape_table_data returns the pointer; a
 * BLS12-381 table or the 256-row layout wrapped by grape_table_from_reference is NOT accepted and,
 * since a raw pointer cannot tell, would be misread), the work runs on the current CUDA device and
 * on `stream` (a cudaStream_t, NULL = default stream).
 *   - calls no cudaMalloc / cudaFree / allocating routine;
 *   - at most 65536 partial sums per call, one or more per (row, window group) where window
 *     groups = ceil(ceil(max_bits / window_bits) / n_windows): rows * groups > 65536 returns
 *     GRAPE_ERR_LIMIT (message from grape_static_error());
 *   - the first call on each device looks up the device address of the static array; issue that
 *     first call outside any stream capture;
 *   - all calls on a device share the array and it keeps the previous call's contents; each call
 *     rewrites what it reads and clears its status word, so calls queued on one stream are safe,
 *     calls that can overlap on the GPU race;
 *   - h_status may be NULL; otherwise the call synchronises `stream` and stores 1 when a scalar
 *     exceeded max_bits, else 0 (with NULL such a scalar goes unreported);
 *   - several host threads may call it: the per-device set-up is serialised and
 *     grape_static_error() returns the calling thread's last message; their kernels still share the
 *     one array, so the overlap rule above applies across threads too.
 * Every GPU that loads the library holds the array until the process exits. */
int grape_commit_i32_static(const void* d_table, uint32_t n_gens, uint32_t window_bits, uint32_t n_windows,
                            const int32_t* d_scalars, uint64_t size, uint32_t wd, uint32_t max_bits,
                            void* d_out, void* stream, uint32_t* h_status);
uint64_t grape_static_scratch_bytes(void);
const char* grape_static_error(void);

/* ---- diagnostics and measurement ----------------------------------------------------------- */
/* Element-wise add (0) / sub (1) / mul (2) over the base field Fp; test hook for the curve code. */
int grape_fp_binary(grape_ctx* ctx, int op, const void* d_a, const void* d_b, void* d_out, uint64_t n);
/* BLS12-381 field hooks (no reference call site): element-wise add (0) / sub (1) / mul (2) over Fr
 * (field 0, 32-byte elements) or Fp (field 1, 48-byte elements); signed int32 -> Fr as
 * grape_fr_from_i32 does for BN254; base-field multiplications per second on register operands. */
int grape_bls12_381_field_binary(grape_ctx* ctx, int field, int op, const void* d_a, const void* d_b,
                                 void* d_out, uint64_t n);
int grape_bls12_381_fr_from_i32(grape_ctx* ctx, const int32_t* d_in, void* d_out, uint64_t n);
int grape_bls12_381_measure_mul_peak(grape_ctx* ctx, double* muls_per_second);
/* Device status word: bit 0 = a scalar exceeded max_bits, bit 1 = lookup query outside its table.
 * Kernels set bits instead of trapping; reading synchronises and clears. */
int grape_ctx_status(grape_ctx* ctx, uint32_t* flags);
/* Kernels launched by this library on the context so far. */
uint64_t grape_ctx_launches(const grape_ctx* ctx);
/* Measured integer-pipe ceilings (operations per second): kind 0 mad.lo.u32, 1 mad.wide.u32,
 * 2 mad.lo.cc/madc.hi pairs (counted as two), 3 Fp Montgomery multiplications, 4 the same with a
 * loop body of 16 inlined multiplications (instruction-fetch probe), 5 dedicated Fp squarings. */
int grape_measure_int_peak(grape_ctx* ctx, int kind, double* ops_per_second);
/* Self-check of the specialised field routines against the plain multiplication (the reference has a
 * dedicated squaring and a Euclid inversion too: include/field/mont_t.cuh:145-192, 1058-1120).
 * field: 0 BN254 Fp, 1 BN254 Fr, 2 BLS12-381 Fp, 3 BLS12-381 Fr; d_elems: n canonical Montgomery
 * elements.  *h_fail_mask = OR over the elements of: 1 squaring != a*a, 2 inverse (batched division
 * steps) != Fermat inverse, 4 a * a^-1 != 1, 8 inverse of 0 != 0, 16 inverse != binary-Euclid inverse. */
int grape_diag_field_check(grape_ctx* ctx, int field, const void* d_elems, uint64_t n, uint32_t* h_fail_mask);
/* Mixed point additions per second on register-resident operands: the commitment kernel's
 * arithmetic with no memory traffic, at the same register budget. */
int grape_measure_madd_peak(grape_ctx* ctx, double* adds_per_second);
/* CUDA-event stopwatch on the context's stream; grape_timer_end synchronises. */
int grape_timer_begin(grape_ctx* ctx);
int grape_timer_end(grape_ctx* ctx, float* ms);
/* Per-kernel timing of the dominant kernel of each call (events around it while enabled). */
int grape_prof_enable(grape_ctx* ctx, int on);
int grape_prof_read(grape_ctx* ctx, float* total_ms, uint32_t* count);
/* Page-locked host memory for the host-buffer entry points. */
int grape_host_alloc_pinned(grape_ctx* ctx, size_t bytes, void** h_out);
int grape_host_free_pinned(grape_ctx* ctx, void* h_ptr);
/* The address at which kernels of this device can read a page-locked host buffer (the buffer itself on
 * systems with unified addressing), or GRAPE_ERR_INVALID when h_ptr is not page-locked.  With it the
 * device-pointer entry points (grape_commit_i32, ...) take their scalars straight from host memory. */
int grape_host_device_pointer(grape_ctx* ctx, const void* h_ptr, void** d_out);

#ifdef __cplusplus
}
#endif
#endif /* GRAPE_B200_H */
