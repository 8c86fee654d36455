// The Fiat-Shamir transcript (Merlin over STROBE-128 / Keccak-f[1600], as wrapped by
// src/util/transcript.rs:13-46) in a form one GPU thread can run, so the last rounds of a
// sumcheck can stay inside a single kernel.  Same state layout as merlin.hpp's Strobe128;
// the functions also compile for the host, where the unit tests check them against the oracle.
#pragma once
#include "ff.cuh"

namespace zk {

struct StrobeState {
  uint64_t lanes[25];  // the 200 state bytes, little-endian
  uint32_t pos, pos_begin, cur_flags, pad;
};

ZK_HD uint64_t rotl64_c(uint64_t x, int n) { return n ? (x << n) | (x >> (64 - n)) : x; }

ZK_HD void keccak_f1600_dev(uint64_t* a) {
  const uint64_t rc[24] = {
      0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808Aull, 0x8000000080008000ull,
      0x000000000000808Bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull,
      0x000000000000008Aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000Aull,
      0x000000008000808Bull, 0x800000000000008Bull, 0x8000000000008089ull, 0x8000000000008003ull,
      0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800Aull, 0x800000008000000Aull,
      0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};
  // rho offsets indexed [x + 5 y]
  const int rot[25] = {0, 1, 62, 28, 27, 36, 44, 6, 55, 20, 3, 10, 43, 25, 39, 41, 45, 15, 21, 8, 18, 2, 61, 56, 14};
  uint64_t s[25];
#pragma unroll
  for (int i = 0; i < 25; i++) s[i] = a[i];
#pragma unroll 1
  for (int round = 0; round < 24; round++) {
    uint64_t c[5], d[5], b[25];
#pragma unroll
    for (int x = 0; x < 5; x++) c[x] = s[x] ^ s[x + 5] ^ s[x + 10] ^ s[x + 15] ^ s[x + 20];
#pragma unroll
    for (int x = 0; x < 5; x++) d[x] = c[(x + 4) % 5] ^ rotl64_c(c[(x + 1) % 5], 1);
#pragma unroll
    for (int i = 0; i < 25; i++) s[i] ^= d[i % 5];
#pragma unroll
    for (int y = 0; y < 5; y++)
#pragma unroll
      for (int x = 0; x < 5; x++) b[y + 5 * ((2 * x + 3 * y) % 5)] = rotl64_c(s[x + 5 * y], rot[x + 5 * y]);
#pragma unroll
    for (int y = 0; y < 5; y++)
#pragma unroll
      for (int x = 0; x < 5; x++) s[x + 5 * y] = b[x + 5 * y] ^ (~b[(x + 1) % 5 + 5 * y] & b[(x + 2) % 5 + 5 * y]);
    s[0] ^= rc[round];
  }
#pragma unroll
  for (int i = 0; i < 25; i++) a[i] = s[i];
}

constexpr uint32_t kStrobeRate = 166;

ZK_HD void strobe_xor_byte(StrobeState& st, uint32_t pos, uint32_t byte) {
  st.lanes[pos >> 3] ^= (uint64_t)(byte & 0xffu) << (8 * (pos & 7));
}
ZK_HD uint32_t strobe_get_byte(const StrobeState& st, uint32_t pos) {
  return (uint32_t)(st.lanes[pos >> 3] >> (8 * (pos & 7))) & 0xffu;
}
ZK_HD void strobe_clear_byte(StrobeState& st, uint32_t pos) {
  st.lanes[pos >> 3] &= ~((uint64_t)0xff << (8 * (pos & 7)));
}
ZK_HD void strobe_run_f(StrobeState& st) {
  strobe_xor_byte(st, st.pos, st.pos_begin);
  strobe_xor_byte(st, st.pos + 1, 0x04);
  strobe_xor_byte(st, kStrobeRate + 1, 0x80);
  keccak_f1600_dev(st.lanes);
  st.pos = 0;
  st.pos_begin = 0;
}
ZK_HD void strobe_absorb(StrobeState& st, const uint8_t* d, uint32_t n) {
  for (uint32_t i = 0; i < n; i++) {
    strobe_xor_byte(st, st.pos++, d[i]);
    if (st.pos == kStrobeRate) strobe_run_f(st);
  }
}
ZK_HD void strobe_begin_op(StrobeState& st, uint32_t flags) {
  const uint8_t hdr[2] = {(uint8_t)st.pos_begin, (uint8_t)flags};
  st.pos_begin = st.pos + 1;
  st.cur_flags = flags;
  strobe_absorb(st, hdr, 2);
  if ((flags & (4u | 32u)) && st.pos != 0) strobe_run_f(st);
}

// Transcript::append_scalar(label, x): meta-AD(label) | meta-AD(len = 32, continued) | AD(32 canonical bytes)
ZK_HD void transcript_append_scalar_dev(StrobeState& st, const char* label, uint32_t label_len, const Fr& mont) {
  const Fr c = from_mont(mont);
  uint8_t bytes[32];
  for (int i = 0; i < 8; i++)
    for (int k = 0; k < 4; k++) bytes[4 * i + k] = (uint8_t)(c.v[i] >> (8 * k));
  const uint8_t len_le[4] = {32, 0, 0, 0};
  strobe_begin_op(st, 16u | 2u);
  strobe_absorb(st, reinterpret_cast<const uint8_t*>(label), label_len);
  strobe_absorb(st, len_le, 4);
  strobe_begin_op(st, 2u);
  strobe_absorb(st, bytes, 32);
}

// Transcript::challenge_scalar(label): 64 PRF bytes, the first 32 reduced mod r (Montgomery out).
ZK_HD Fr transcript_challenge_scalar_dev(StrobeState& st, const char* label, uint32_t label_len) {
  const uint8_t len_le[4] = {64, 0, 0, 0};
  strobe_begin_op(st, 16u | 2u);
  strobe_absorb(st, reinterpret_cast<const uint8_t*>(label), label_len);
  strobe_absorb(st, len_le, 4);
  strobe_begin_op(st, 1u | 2u | 4u);
  Fr raw = Fr::zero();
  for (uint32_t i = 0; i < 64; i++) {
    const uint32_t b = strobe_get_byte(st, st.pos);
    strobe_clear_byte(st, st.pos);
    st.pos++;
    if (i < 32) raw.v[i >> 2] |= b << (8 * (i & 3));
    if (st.pos == kStrobeRate) strobe_run_f(st);
  }
  return to_mont(raw);
}

}  // namespace zk
