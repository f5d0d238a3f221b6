// Harness that drives the REFERENCE's own library (its unmodified src/*.cu, compiled against the
// libff stand-in in oracle/ref_shim) so that its outputs can pin the oracle and this repository's
// kernels, and so that its commitment kernel can be timed on the same GPU.
// TEST INFRASTRUCTURE ONLY.  Built by oracle/Makefile into oracle/_ref/ (never committed).
//
//   ref_harness parity <in.bin> <out.bin>     commit / open / prove_matmul / tLookupRange on given data
//   ref_harness commit-bench <rows> <steps>   times Hyrax::commit(int*) on int16-range rows of 4096
//   ref_harness matmul-bench <shrink> <steps> times prove_matmul on (2048/shrink) x 4096 . (4096/shrink) x 4096
//   ref_harness lookup-bench <log2 D> <steps> times tLookupRange::prove on 2^D queries into a 2^16 table
//
// Shapes are restricted to what the reference's kernels handle without reading out of bounds
// (they have no guards): rows a multiple of 32, power-of-two sizes.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "Hyrax.cuh"
#include "prove.cuh"
#include "tlookup.cuh"

template <class T>
static void put(std::vector<unsigned char>& out, const T* p, size_t n) {
  const unsigned char* b = reinterpret_cast<const unsigned char*>(p);
  out.insert(out.end(), b, b + n * sizeof(T));
}

template <class T>
static T* to_dev(const T* h, size_t n) {
  T* d;
  cudaMalloc(&d, n * sizeof(T));
  cudaMemcpy(d, h, n * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}

static int parity(const char* in_path, const char* out_path) {
  FILE* f = fopen(in_path, "rb");
  if (!f) return 3;
  uint32_t hdr[10];
  if (fread(hdr, 4, 10, f) != 10) return 4;
  const uint32_t n_gens = hdr[0], size = hdr[1], N = hdr[2], layer_num = hdr[3], L = hdr[4], Nn = hdr[5], M = hdr[6],
                 K = hdr[7], lk_len = hdr[8], lk_D = hdr[9];
  std::vector<int> tensor(size), A((size_t)L * Nn * K), B((size_t)L * M * K), Y((size_t)L * Nn * M), Q(lk_D);
  if (fread(tensor.data(), 4, tensor.size(), f) != tensor.size() || fread(A.data(), 4, A.size(), f) != A.size() ||
      fread(B.data(), 4, B.size(), f) != B.size() || fread(Y.data(), 4, Y.size(), f) != Y.size() ||
      fread(Q.data(), 4, Q.size(), f) != Q.size())
    return 5;
  // second part: Hadamard product, claim batching, mapping lookup
  uint32_t hdr2[6];
  if (fread(hdr2, 4, 6, f) != 6) return 4;
  const uint32_t eL = hdr2[0], eM = hdr2[1], eN = hdr2[2], map_len = hdr2[3], map_D = hdr2[4];
  const int map_low = (int)hdr2[5];
  const size_t esize = (size_t)eL * eM * eN;
  std::vector<int> EA(esize), EB(esize), MIN(map_D), MOUT(map_D);
  if (fread(EA.data(), 4, esize, f) != esize || fread(EB.data(), 4, esize, f) != esize ||
      fread(MIN.data(), 4, map_D, f) != map_D || fread(MOUT.data(), 4, map_D, f) != map_D)
    return 5;
  fclose(f);
  std::vector<unsigned char> out;
  ppT::init_public_params();
  ref_shim_seed(99);
  // test/ppgen.cu: generators and the 256-row table
  affine_t* points;
  cudaMalloc(&points, sizeof(affine_t) * (size_t)n_gens * 256);
  std::vector<bn128> cpu_points = precompute_generators(n_gens, 256, points);
  cudaDeviceSynchronize();
  put(out, cpu_points.data(), cpu_points.size());
  // test/HyraxTest.cu
  int* d_tensor = to_dev(tensor.data(), tensor.size());
  Hyrax hyrax(layer_num, n_gens / 16, points, cpu_points[0]);
  FrTensor fr_tensor(size, d_tensor);
  jacob_t* c0 = hyrax.commit(d_tensor, size, N);
  jacob_t* c1 = hyrax.commit(fr_tensor, size, N);
  const uint rows = size / (N * 16);
  std::vector<jacob_t> h0(rows), h1(rows);
  cudaMemcpy(h0.data(), c0, rows * sizeof(jacob_t), cudaMemcpyDeviceToHost);
  cudaMemcpy(h1.data(), c1, rows * sizeof(jacob_t), cudaMemcpyDeviceToHost);
  put(out, h0.data(), rows);
  put(out, h1.data(), rows);
  std::vector<Fr> eval_point = random_vec(Log2(size));
  Fr cc = Fr::random_element();
  Hyrax_proof proof = hyrax.open(fr_tensor, eval_point, cc, size, N);
  put(out, &proof.result, 1);
  put(out, proof.z, proof.z_size);
  put(out, &proof.commit_d, 1);
  put(out, &proof.commit_ad, 1);
  // test/matmul.cu
  int* dA = to_dev(A.data(), A.size());
  int* dB = to_dev(B.data(), B.size());
  int* dY = to_dev(Y.data(), Y.size());
  FrTensor x(A.size(), dA), w(B.size(), dB), y(Y.size(), dY);
  std::vector<Fr> u = random_vec(Log2(Y.size())), v = random_vec(Log2(K * L));
  Fr claim = y(u);
  Fr claim0 = claim;
  auto pr = prove_matmul(x, w, L, Nn, M, K, u, v, claim);
  put(out, &claim0, 1);
  put(out, &pr.first, 1);
  put(out, &pr.second, 1);
  put(out, &claim, 1);
  // test/tlookupTest.cu
  int* dQ = to_dev(Q.data(), Q.size());
  tLookupRange rs(-(int)(lk_len / 2), lk_len);
  FrTensor x_tensor(lk_D, dQ), lookup_A(lk_D);
  std::vector<Fr> lv = random_vec(Log2(lk_D));
  double com_time = 0.0;
  Fr value = rs.prove(x_tensor, lookup_A, lv, hyrax, n_gens / 16, com_time);
  put(out, &value, 1);
  // prove_eleMul (test/eleWiseMul.cu flow): claim = (A.B)~(u)
  {
    int* dEA = to_dev(EA.data(), esize);
    int* dEB = to_dev(EB.data(), esize);
    FrTensor ea(esize, dEA), eb(esize, dEB);
    FrTensor prod(ea);
    prod *= eb;
    std::vector<Fr> eu = random_vec(Log2(esize)), ev = random_vec(Log2(esize));
    Fr ecl = prod(eu);
    Fr ecl0 = ecl;
    auto ep = prove_eleMul(ea, eb, eL, eM, eN, eu, ev, ecl);
    put(out, &ecl0, 1);
    put(out, &ep.first, 1);
    put(out, &ep.second, 1);
    // combine_claims (test/combine_value.cu flow) on the first factor, two points
    FrTensor X(esize, dEA);
    std::vector<Fr> u1 = random_vec(Log2(esize)), u2 = random_vec(Log2(esize)), cv = random_vec(Log2(esize));
    FrTensor t1(X), t2(X);
    Fr c1 = t1(u1), c2 = t2(u2);
    Fr comb = combine_claims(X, {c1, c2}, {u1, u2}, cv, esize);
    put(out, &c1, 1);
    put(out, &c2, 1);
    put(out, &comb, 1);
  }
  // tLookupRangeMapping (test/tlookupMapTest.cu flow); the table file was written by the caller
  {
    std::string table_path = std::string(in_path) + ".table";
    tLookupRangeMapping mp(map_low, map_len, table_path);
    int* dIN = to_dev(MIN.data(), map_D);
    int* dOUT = to_dev(MOUT.data(), map_D);
    FrTensor s_in(map_D, dIN), s_out(map_D, dOUT), mA(map_D);
    std::vector<Fr> mv = random_vec(Log2(map_D));
    double com_time = 0.0;
    Fr mval = mp.prove(s_in, s_out, mA, mv, hyrax, n_gens / 16, com_time);
    put(out, &mp.r, 1);
    put(out, &mval, 1);
  }
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(e));
    return 6;
  }
  f = fopen(out_path, "wb");
  fwrite(out.data(), 1, out.size(), f);
  fclose(f);
  return 0;
}

static int commit_bench(uint32_t rows, int steps, int warmup) {
  const uint32_t wd = 4096, n_gens = 4096;
  ppT::init_public_params();
  ref_shim_seed(0xC4);
  affine_t* points;
  cudaMalloc(&points, sizeof(affine_t) * (size_t)n_gens * 256);
  auto t0 = std::chrono::high_resolution_clock::now();
  std::vector<bn128> cpu_points = precompute_generators(n_gens, 256, points);
  cudaDeviceSynchronize();
  double table_s = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
  std::mt19937 rng(7);
  std::normal_distribution<float> dist(0.f, 0.02f * 65536.f);
  std::vector<int> h((size_t)rows * wd);
  for (auto& x : h) {
    float v = std::round(dist(rng));
    x = (int)std::min(32767.f, std::max(-32768.f, v));
  }
  int* d = to_dev(h.data(), h.size());
  Hyrax hyrax(1, n_gens / 16, points, cpu_points[0]);
  jacob_t* c = nullptr;
  for (int s = 0; s < (warmup < 1 ? 1 : warmup); s++) {  // untimed warm-up steps
    c = hyrax.commit(d, rows * wd, wd / 16);
    cudaFree(c);
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int s = 0; s < steps; s++) {
    c = hyrax.commit(d, rows * wd, wd / 16);
    cudaFree(c);
  }
  cudaEventRecord(e1);
  cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  // the same with the reference's own data movement around it: pageable host tensor -> device
  // (load_data, src/ioutils.cu:105-124), commit, commitments back to the host (savebin, :3-40)
  std::vector<jacob_t> h_out(rows);
  cudaEventRecord(e0);
  for (int s = 0; s < steps; s++) {
    cudaMemcpy(d, h.data(), h.size() * sizeof(int), cudaMemcpyHostToDevice);
    c = hyrax.commit(d, rows * wd, wd / 16);
    cudaMemcpy(h_out.data(), c, rows * sizeof(jacob_t), cudaMemcpyDeviceToHost);
    cudaFree(c);
  }
  cudaEventRecord(e1);
  cudaEventSynchronize(e1);
  float ms_e2e = 0;
  cudaEventElapsedTime(&ms_e2e, e0, e1);
  cudaError_t e = cudaGetLastError();
  printf("{\"rows\": %u, \"row_len\": %u, \"warmup\": %d, \"steps\": %d, \"ms_per_step\": %.4f, \"points_per_s\": %.1f, "
         "\"e2e_ms_per_step\": %.4f, \"e2e_points_per_s\": %.1f, \"table_build_s\": %.3f, \"cuda_status\": \"%s\"}\n",
         rows, wd, warmup < 1 ? 1 : warmup, steps, ms / steps, (double)rows * wd * steps / (ms * 1e-3), ms_e2e / steps,
         (double)rows * wd * steps / (ms_e2e * 1e-3), table_s, cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 6;
}

// C2: the reference's prove_matmul on A [N][K], B [M][K] with K = 4096 (test/matmul.cu flow; the
// claim is formed with the reference's own folds instead of a host matrix product).
static int matmul_bench(uint32_t shrink, int steps) {
  const uint32_t L = 1, N = 2048 / shrink, M = 4096 / shrink, K = 4096;
  ppT::init_public_params();
  ref_shim_seed(0xC2);
  std::mt19937 rng(11);
  std::normal_distribution<float> dist(0.f, 0.02f * 65536.f);
  std::vector<int> hA((size_t)N * K), hB((size_t)M * K);
  for (auto& x : hA) x = (int)std::round(dist(rng));
  for (auto& x : hB) x = (int)std::round(dist(rng));
  int* dA = to_dev(hA.data(), hA.size());
  int* dB = to_dev(hB.data(), hB.size());
  std::vector<Fr> u = random_vec(Log2(L * N * M)), v = random_vec(Log2(K * L));
  Fr claim0;
  {
    FrTensor a2(hA.size(), dA), b2(hB.size(), dB);
    fr_t* U;
    cudaMalloc(&U, sizeof(fr_t) * u.size());
    cudaMemcpy(U, u.data(), sizeof(fr_t) * u.size(), cudaMemcpyHostToDevice);
    a2.partial_eval(a2.size, U, N, Log2(M), K);
    b2.partial_eval(b2.size, U, M, 0, K);
    FrTensor a(K), b(K);
    cudaMemcpy(a.gpu_data, a2.gpu_data, sizeof(fr_t) * K, cudaMemcpyDeviceToDevice);
    cudaMemcpy(b.gpu_data, b2.gpu_data, sizeof(fr_t) * K, cudaMemcpyDeviceToDevice);
    a *= b;
    claim0 = a.sum(K);
    cudaFree(U);
  }
  double total = 0;
  for (int s = 0; s < steps + 1; s++) {
    FrTensor x(hA.size(), dA), w(hB.size(), dB);
    Fr claim = claim0;
    cudaDeviceSynchronize();
    auto t0 = std::chrono::high_resolution_clock::now();
    auto pr = prove_matmul(x, w, L, N, M, K, u, v, claim);
    cudaDeviceSynchronize();
    double dt = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
    if (s > 0) total += dt;  // first call is the warm-up
    (void)pr;
  }
  cudaError_t e = cudaGetLastError();
  printf("{\"N\": %u, \"M\": %u, \"K\": %u, \"steps\": %d, \"ms_per_proof\": %.4f, \"cuda_status\": \"%s\"}\n", N, M, K,
         steps, total / steps * 1e3, cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 6;
}

// C3: the reference's tLookupRange::prove on 2^log2_d uniform queries into a 2^16 table, with its
// commitments of A and m over 4096 generators (test/tlookupTest.cu flow).
static int lookup_bench(uint32_t log2_d, int steps, uint32_t n_gens) {
  const uint32_t D = 1u << log2_d, len = 1u << 16;
  ppT::init_public_params();
  ref_shim_seed(0xC3);
  affine_t* points;
  cudaMalloc(&points, sizeof(affine_t) * (size_t)n_gens * 256);
  std::vector<bn128> cpu_points = precompute_generators(n_gens, 256, points);
  cudaDeviceSynchronize();
  Hyrax hyrax(1, n_gens / 16, points, cpu_points[0]);
  std::mt19937 rng(13);
  std::uniform_int_distribution<int> dist(-(int)(len / 2), (int)(len / 2) - 1);
  std::vector<int> hq(D);
  for (auto& x : hq) x = dist(rng);
  int* dQ = to_dev(hq.data(), hq.size());
  std::vector<Fr> v = random_vec(Log2(D));
  double total = 0, com_total = 0;
  for (int s = 0; s < steps + 1; s++) {
    tLookupRange rs(-(int)(len / 2), len);
    FrTensor x_tensor(D, dQ), A(D);
    double com_time = 0.0;
    cudaDeviceSynchronize();
    auto t0 = std::chrono::high_resolution_clock::now();
    Fr value = rs.prove(x_tensor, A, v, hyrax, n_gens / 16, com_time);
    cudaDeviceSynchronize();
    double dt = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
    if (s > 0) {
      total += dt;
      com_total += com_time;
    }
    (void)value;
  }
  cudaError_t e = cudaGetLastError();
  printf("{\"D\": %u, \"table\": %u, \"generators\": %u, \"steps\": %d, \"ms_per_proof\": %.4f, \"commit_ms_reported_by_reference\": %.4f, "
         "\"cuda_status\": \"%s\"}\n", D, len, n_gens, steps, total / steps * 1e3, com_total / steps * 1e3, cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 6;
}

int main(int argc, char** argv) {
  if (argc >= 4 && std::string(argv[1]) == "parity") return parity(argv[2], argv[3]);
  if (argc >= 4 && std::string(argv[1]) == "commit-bench") return commit_bench(atoi(argv[2]), atoi(argv[3]), argc >= 5 ? atoi(argv[4]) : 1);
  if (argc >= 4 && std::string(argv[1]) == "matmul-bench") return matmul_bench(atoi(argv[2]), atoi(argv[3]));
  if (argc >= 4 && std::string(argv[1]) == "lookup-bench") return lookup_bench(atoi(argv[2]), atoi(argv[3]), argc >= 5 ? (uint32_t)atoi(argv[4]) : 4096u);
  fprintf(stderr, "usage: ref_harness parity <in> <out> | commit-bench <rows> <steps> [warm-up steps] | matmul-bench <shrink> <steps> | "
                  "lookup-bench <log2 queries> <steps> [generators]\n");
  return 2;
}
