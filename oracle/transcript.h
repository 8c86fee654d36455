/* CPU oracle (TEST INFRASTRUCTURE ONLY): the reference's Transcript (src/util/transcript.rs:13-46)
 * over merlin 3.0.0, which is not vendored with the reference.  Restated from the STROBE-128
 * v1.0.2 and Merlin v1.0 specifications with a table-driven Keccak-f[1600] (FIPS 202). */
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>
#include "field.h"

namespace orc {

inline void keccakf(uint64_t st[25]) {
  static const uint64_t rc[24] = {
      0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808aull, 0x8000000080008000ull,
      0x000000000000808bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull,
      0x000000000000008aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000aull,
      0x000000008000808bull, 0x800000000000008bull, 0x8000000000008089ull, 0x8000000000008003ull,
      0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800aull, 0x800000008000000aull,
      0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};
  static const int rot[5][5] = {{0, 36, 3, 41, 18}, {1, 44, 10, 45, 2}, {62, 6, 43, 15, 61}, {28, 55, 25, 21, 56}, {27, 20, 39, 8, 14}};
  for (int r = 0; r < 24; r++) {
    uint64_t c[5], b[25];
    for (int x = 0; x < 5; x++) c[x] = st[x] ^ st[x + 5] ^ st[x + 10] ^ st[x + 15] ^ st[x + 20];
    for (int x = 0; x < 5; x++) {
      const uint64_t t = c[(x + 1) % 5];
      const uint64_t d = c[(x + 4) % 5] ^ ((t << 1) | (t >> 63));
      for (int y = 0; y < 5; y++) st[x + 5 * y] ^= d;
    }
    for (int x = 0; x < 5; x++)
      for (int y = 0; y < 5; y++) {
        const int s = rot[x][y];
        const uint64_t v = st[x + 5 * y];
        b[y + 5 * ((2 * x + 3 * y) % 5)] = s ? (v << s) | (v >> (64 - s)) : v;
      }
    for (int y = 0; y < 5; y++)
      for (int x = 0; x < 5; x++) st[x + 5 * y] = b[x + 5 * y] ^ (~b[(x + 1) % 5 + 5 * y] & b[(x + 2) % 5 + 5 * y]);
    st[0] ^= rc[r];
  }
}

class Transcript {
 public:
  explicit Transcript(const std::string& label) {
    memset(st, 0, 200);
    const uint8_t h[6] = {1, 168, 1, 0, 1, 96};
    memcpy(st, h, 6);
    memcpy(st + 6, "STROBEv1.0.2", 12);
    perm();
    pos = pos_begin = 0;
    meta("Merlin v1.0", 11, false);
    append_message("dom-sep", (const uint8_t*)label.data(), label.size());
  }
  void append_message(const char* label, const uint8_t* m, size_t n) {
    uint8_t le[4] = {(uint8_t)n, (uint8_t)(n >> 8), (uint8_t)(n >> 16), (uint8_t)(n >> 24)};
    meta(label, strlen(label), false);
    meta(le, 4, true);
    begin(2, false);
    absorb(m, n);
  }
  void append_u64(const char* label, uint64_t v) {
    uint8_t le[8];
    for (int i = 0; i < 8; i++) le[i] = (uint8_t)(v >> (8 * i));
    append_message(label, le, 8);
  }
  void challenge_bytes(const char* label, uint8_t* out, size_t n) {
    uint8_t le[4] = {(uint8_t)n, (uint8_t)(n >> 8), (uint8_t)(n >> 16), (uint8_t)(n >> 24)};
    meta(label, strlen(label), false);
    meta(le, 4, true);
    begin(1 | 2 | 4, false);
    for (size_t i = 0; i < n; i++) {
      out[i] = st[pos];
      st[pos++] = 0;
      if (pos == 166) runf();
    }
  }
  // append_scalar: 32-byte canonical little-endian (util/poly.rs:79-83)
  void append_scalar(const char* label, const Fr& x) {
    uint64_t c[4];
    x.to_canonical(c);
    append_message(label, (const uint8_t*)c, 32);
  }
  // challenge_scalar: 64 bytes drawn, first 32 reduced mod r (transcript.rs:38-42, poly.rs:72-78)
  Fr challenge_scalar(const char* label) {
    uint8_t buf[64];
    challenge_bytes(label, buf, 64);
    uint64_t c[4];
    memcpy(c, buf, 32);
    return Fr::from_canonical(c);
  }

 private:
  uint8_t st[200];
  int pos, pos_begin;
  void perm() {
    uint64_t w[25];
    memcpy(w, st, 200);
    keccakf(w);
    memcpy(st, w, 200);
  }
  void runf() {
    st[pos] ^= (uint8_t)pos_begin;
    st[pos + 1] ^= 0x04;
    st[167] ^= 0x80;
    perm();
    pos = pos_begin = 0;
  }
  void absorb(const uint8_t* d, size_t n) {
    for (size_t i = 0; i < n; i++) {
      st[pos++] ^= d[i];
      if (pos == 166) runf();
    }
  }
  void begin(uint8_t flags, bool more) {
    if (more) return;
    const uint8_t hdr[2] = {(uint8_t)pos_begin, flags};
    pos_begin = pos + 1;
    absorb(hdr, 2);
    if ((flags & (4 | 32)) && pos != 0) runf();
  }
  void meta(const void* d, size_t n, bool more) {
    begin(16 | 2, more);
    absorb((const uint8_t*)d, n);
  }
};
}  // namespace orc
