// A driver in the style of the reference's test/HyraxTest.cu, test/matmul.cu and test/tlookupTest.cu,
// written against include/grape_veneer.hpp only.  It reads its inputs from a blob prepared by the
// test (generator table in the reference's points.bin layout, tensors), runs commit / open /
// prove_matmul / tLookupRange::prove with a seeded random stream and writes every result to a
// blob that the test compares with the oracle.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "grape_veneer.hpp"

template <class T>
static void put(std::vector<unsigned char>& out, const T* p, size_t n) {
  const unsigned char* b = reinterpret_cast<const unsigned char*>(p);
  out.insert(out.end(), b, b + n * sizeof(T));
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  FILE* f = fopen(argv[1], "rb");
  if (!f) return 3;
  uint32_t hdr[10];
  if (fread(hdr, 4, 10, f) != 10) return 4;
  const uint32_t n_gens = hdr[0], size = hdr[1], N = hdr[2], layer_num = hdr[3], L = hdr[4], Nn = hdr[5], M = hdr[6],
                 K = hdr[7], lk_len = hdr[8], lk_D = hdr[9];
  std::vector<affine_t> table(256 * (size_t)n_gens);
  bn128 G;
  std::vector<int> tensor(size), A((size_t)L * Nn * K), B((size_t)L * M * K), Y((size_t)L * Nn * M), Q(lk_D);
  if (fread(table.data(), 64, table.size(), f) != table.size()) return 5;
  if (fread(G.v, 96, 1, f) != 1) return 5;
  if (fread(tensor.data(), 4, tensor.size(), f) != tensor.size()) return 5;
  if (fread(A.data(), 4, A.size(), f) != A.size() || fread(B.data(), 4, B.size(), f) != B.size() ||
      fread(Y.data(), 4, Y.size(), f) != Y.size() || fread(Q.data(), 4, Q.size(), f) != Q.size())
    return 5;
  fclose(f);
  std::vector<unsigned char> out;
  try {
    grape_ctx* c = grape_veneer::ctx();
    grape_rng_seed(c, 99);
    auto to_dev = [&](const void* h, size_t bytes) {
      void* d = grape_veneer::dev_alloc(bytes);
      grape_veneer::check(grape_h2d(c, d, h, bytes));
      grape_veneer::check(grape_ctx_sync(c));
      return d;
    };
    // ---- test/HyraxTest.cu flow ---------------------------------------------------------------
    affine_t* points = (affine_t*)to_dev(table.data(), table.size() * 64);
    int* d_tensor = (int*)to_dev(tensor.data(), tensor.size() * 4);
    Hyrax hyrax(layer_num, n_gens / 16, points, G);
    FrTensor fr_tensor(size, d_tensor);
    jacob_t* commitment = hyrax.commit(d_tensor, size, N);
    jacob_t* commitment1 = hyrax.commit(fr_tensor, size, N);
    const uint rows = size / (N * 16);
    std::vector<jacob_t> h_com(rows), h_com1(rows);
    grape_veneer::check(grape_d2h(c, h_com.data(), commitment, rows * 96));
    grape_veneer::check(grape_d2h(c, h_com1.data(), commitment1, rows * 96));
    put(out, h_com.data(), rows);
    put(out, h_com1.data(), rows);
    std::vector<Fr> eval_point = random_vec(Log2(size));
    Fr cc = Fr::random_element();
    Hyrax_proof proof = hyrax.open(fr_tensor, eval_point, cc, size, N);
    put(out, &proof.result, 1);
    put(out, proof.z, proof.z_size);
    put(out, &proof.commit_d, 1);
    put(out, &proof.commit_ad, 1);
    // ---- test/matmul.cu flow -------------------------------------------------------------------
    int* dA = (int*)to_dev(A.data(), A.size() * 4);
    int* dB = (int*)to_dev(B.data(), B.size() * 4);
    int* dY = (int*)to_dev(Y.data(), Y.size() * 4);
    FrTensor x(A.size(), dA), w(B.size(), dB), y(Y.size(), dY);
    std::vector<Fr> u = random_vec(Log2(Y.size())), v = random_vec(Log2(K * L));
    Fr claim = y(u);
    Fr claim0 = claim;
    auto pr = prove_matmul(x, w, L, Nn, M, K, u, v, claim);
    put(out, &claim0, 1);
    put(out, &pr.first, 1);
    put(out, &pr.second, 1);
    put(out, &claim, 1);
    // a wrong claim must throw, as the reference does
    {
      FrTensor x2(A.size(), dA), w2(B.size(), dB);
      Fr bad = claim0 + Fr::one();
      bool threw = false;
      try {
        prove_matmul(x2, w2, L, Nn, M, K, u, v, bad);
      } catch (const std::runtime_error&) {
        threw = true;
      }
      uint32_t flag = threw;
      put(out, &flag, 1);
    }
    // ---- test/tlookupTest.cu flow ---------------------------------------------------------------
    int* dQ = (int*)to_dev(Q.data(), Q.size() * 4);
    tLookupRange rs(-(int)(lk_len / 2), lk_len);
    FrTensor x_tensor(lk_D, dQ), lookup_A(lk_D);
    std::vector<Fr> lv = random_vec(Log2(lk_D));
    double com_time = 0.0;
    Fr value = rs.prove(x_tensor, lookup_A, lv, hyrax, n_gens / 16, com_time);
    put(out, &value, 1);
    // claim algebra of the rescaling step (test/llm.cu:108): q * 2^16 + rem
    Fr combined = pr.first * Fr(1L << 16) + value;
    put(out, &combined, 1);
    grape_dev_free(c, commitment);
    grape_dev_free(c, commitment1);
  } catch (const std::exception& e) {
    fprintf(stderr, "driver failed: %s\n", e.what());
    return 1;
  }
  f = fopen(argv[2], "wb");
  fwrite(out.data(), 1, out.size(), f);
  fclose(f);
  return 0;
}
