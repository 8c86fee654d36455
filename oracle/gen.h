/* CPU oracle (TEST INFRASTRUCTURE ONLY): the seeded input streams of the benchmark on the host, so that the
 * CPU arm can run on exactly the bytes the GPU arm generates on the device.  ChaCha20 (RFC 8439 block
 * function, zero nonce, 32-bit block counter), key = seed | stream as two little-endian u64 then zeros;
 * block i defines element i:  uniform = the 64 keystream bytes as a 512-bit little-endian integer mod r;
 * small = (keystream word 0, low `bits` bits) - 2^(bits-1), negatives lifted to r - |v|. */
#pragma once
#include "poly.h"

namespace orc {

inline uint32_t rotl32(uint32_t v, int n) { return (v << n) | (v >> (32 - n)); }

inline void chacha_block(uint64_t seed, uint64_t stream, uint32_t counter, uint32_t out[16]) {
  const uint32_t st[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, (uint32_t)seed, (uint32_t)(seed >> 32),
                           (uint32_t)stream, (uint32_t)(stream >> 32), 0, 0, 0, 0, counter, 0, 0, 0};
  uint32_t x[16];
  for (int i = 0; i < 16; i++) x[i] = st[i];
  auto qr = [&](int a, int b, int c, int d) {
    x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 16);
    x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 12);
    x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 8);
    x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 7);
  };
  for (int r = 0; r < 10; r++) {
    qr(0, 4, 8, 12); qr(1, 5, 9, 13); qr(2, 6, 10, 14); qr(3, 7, 11, 15);
    qr(0, 5, 10, 15); qr(1, 6, 11, 12); qr(2, 7, 8, 13); qr(3, 4, 9, 14);
  }
  for (int i = 0; i < 16; i++) out[i] = x[i] + st[i];
}

inline void gen_uniform(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, uint64_t* out) {
  uint64_t two256[4] = {0, 0, 0, 0};
  // 2^256 mod r in Montgomery form: from_canonical(1) is R = 2^256 mod r as an element; its Montgomery
  // form is what multiplying by it needs
  uint64_t one[4] = {1, 0, 0, 0};
  const Fr r_elem = Fr::from_canonical(one);  // the element 1, limbs = R mod r
  memcpy(two256, r_elem.l, 32);               // the integer R mod r
  const Fr shift = Fr::from_canonical(two256);  // the element 2^256 mod r
  parallel_for(count, [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; i++) {
      uint32_t ks[16];
      chacha_block(seed, stream, (uint32_t)(start + i), ks);
      uint64_t lo[4], hi[4];
      for (int k = 0; k < 4; k++) {
        lo[k] = (uint64_t)ks[2 * k] | ((uint64_t)ks[2 * k + 1] << 32);
        hi[k] = (uint64_t)ks[8 + 2 * k] | ((uint64_t)ks[8 + 2 * k + 1] << 32);
      }
      const Fr v = Fr::from_canonical(lo) + Fr::from_canonical(hi) * shift;
      memcpy(out + 4 * i, v.l, 32);
    }
  });
}

inline void gen_small(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int bits, uint64_t* out) {
  parallel_for(count, [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; i++) {
      uint32_t ks[16];
      chacha_block(seed, stream, (uint32_t)(start + i), ks);
      const int64_t sv = (int64_t)(ks[0] & ((1u << bits) - 1u)) - (int64_t)(1u << (bits - 1));
      Fr v = Fr::from_u64((uint64_t)(sv < 0 ? -sv : sv));
      if (sv < 0) v = v.neg();
      memcpy(out + 4 * i, v.l, 32);
    }
  });
}

}  // namespace orc
