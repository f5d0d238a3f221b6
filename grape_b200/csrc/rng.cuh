// The prover's randomness (Hyrax blinding vectors, the lookups' alpha / r / u): the stand-in for
// libff's Fr::random_element(), which the reference calls for every one of them
// (src/Hyrax.cu:253-256, src/tlookup.cu:247,293,351, src/ec_operation.cu:55).
//
// Two sources, chosen per context:
//   * default: ChaCha20 in counter mode under a 256-bit key the context draws from the operating
//     system's generator when it is created.  Element i of the stream is block i of the cipher: 64
//     bytes, read as a 512-bit integer and reduced mod r (bias below 2^-250).  Blocks are
//     independent, so the device fills a whole blinding vector in one launch.
//   * after grape_rng_seed: a SplitMix64 stream with 64 bits of state, identical to the oracle's.
//     It exists so that tests and parity runs can replay the reference's draws; it is NOT fit for
//     proofs whose zero-knowledge matters (z = c x + d reveals x when d is predictable).
#pragma once
#include <cstdint>

#include "hostfr.hpp"

namespace grape {

#if defined(__CUDACC__)
#define GRAPE_HD __host__ __device__
#else
#define GRAPE_HD
#endif

GRAPE_HD inline uint32_t rotl32(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }

// One ChaCha20 block (RFC 8439 layout: constants, 8 key words, 32-bit block counter, 3 nonce words;
// here the 64-bit stream position fills the counter and the first nonce word, the rest of the nonce
// is zero).
GRAPE_HD inline void chacha20_block(const uint32_t key[8], uint64_t position, uint32_t out[16]) {
  uint32_t s[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key[0], key[1], key[2], key[3],
                    key[4],      key[5],      key[6],      key[7],      (uint32_t)position, (uint32_t)(position >> 32), 0u, 0u};
  uint32_t x[16];
  for (int i = 0; i < 16; i++) x[i] = s[i];
#define GRAPE_QR(a, b, c, d)                  \
  x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 16); \
  x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 12); \
  x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 8);  \
  x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 7);
  for (int r = 0; r < 10; r++) {
    GRAPE_QR(0, 4, 8, 12) GRAPE_QR(1, 5, 9, 13) GRAPE_QR(2, 6, 10, 14) GRAPE_QR(3, 7, 11, 15)
    GRAPE_QR(0, 5, 10, 15) GRAPE_QR(1, 6, 11, 12) GRAPE_QR(2, 7, 8, 13) GRAPE_QR(3, 4, 9, 14)
  }
#undef GRAPE_QR
  for (int i = 0; i < 16; i++) out[i] = x[i] + s[i];
}

struct RngKey {
  uint32_t k[8];
};

// Random-stream state of a context.
struct RngState {
  bool seeded = false;        // false: ChaCha20 under `key`; true: the SplitMix64 test stream
  RngKey key{};               // from the operating system
  uint64_t position = 0;      // next ChaCha20 block
  uint64_t splitmix = 0;      // SplitMix64 state
};

// 512 bits (sixteen little-endian 32-bit words) -> Montgomery residue of the value mod r.
inline HostFr fr_from_512(const uint32_t w[16]) {
  using namespace hostfr_detail;
  uint64_t lo[4], hi[4];
  for (int i = 0; i < 4; i++) {
    lo[i] = (uint64_t)w[2 * i] | ((uint64_t)w[2 * i + 1] << 32);
    hi[i] = (uint64_t)w[8 + 2 * i] | ((uint64_t)w[8 + 2 * i + 1] << 32);
  }
  HostFr r2{{R2[0], R2[1], R2[2], R2[3]}};
  return fr_add(fr_from_raw(lo), fr_mul(fr_from_raw(hi), r2));
}

// The next element of the context's stream (host side).
inline HostFr rng_draw_fr(RngState& st) {
  if (st.seeded) return rng_next_fr(st.splitmix);
  uint32_t blk[16];
  chacha20_block(st.key.k, st.position++, blk);
  return fr_from_512(blk);
}

// Fills key from the operating system's generator; false when none could be read.
bool rng_os_key(RngKey* key);

}  // namespace grape
