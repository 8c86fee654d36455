// Host-side Fiat-Shamir transcript: Merlin (STROBE-128 over Keccak-f[1600]) as wrapped by
// src/util/transcript.rs:13-46 of the reference.  Written from the STROBE v1.0.2 and Merlin
// v1.0 specifications; only the three STROBE operations Merlin uses are present.
#pragma once
#include <cstdint>
#include <cstring>
#include <cstddef>

namespace zk {

inline uint64_t rotl64(uint64_t x, int n) { return n ? (x << n) | (x >> (64 - n)) : x; }

inline void keccak_f1600(uint64_t a[25]) {
  static const uint64_t RC[24] = {
      0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808Aull, 0x8000000080008000ull,
      0x000000000000808Bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull,
      0x000000000000008Aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000Aull,
      0x000000008000808Bull, 0x800000000000008Bull, 0x8000000000008089ull, 0x8000000000008003ull,
      0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800Aull, 0x800000008000000Aull,
      0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};
  // rho offsets and pi destinations generated from the (x, y) -> (y, 2x + 3y) walk
  for (int round = 0; round < 24; round++) {
    uint64_t c[5], d[5];
    for (int x = 0; x < 5; x++) c[x] = a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20];
    for (int x = 0; x < 5; x++) d[x] = c[(x + 4) % 5] ^ rotl64(c[(x + 1) % 5], 1);
    for (int i = 0; i < 25; i++) a[i] ^= d[i % 5];
    // rho + pi: follow the single 24-cycle starting at (1, 0)
    int x = 1, y = 0;
    uint64_t cur = a[1];
    for (int t = 0; t < 24; t++) {
      const int nx = y, ny = (2 * x + 3 * y) % 5;
      const uint64_t tmp = a[nx + 5 * ny];
      a[nx + 5 * ny] = rotl64(cur, ((t + 1) * (t + 2) / 2) % 64);
      cur = tmp;
      x = nx;
      y = ny;
    }
    for (int row = 0; row < 25; row += 5) {
      uint64_t r[5];
      for (int k = 0; k < 5; k++) r[k] = a[row + k];
      for (int k = 0; k < 5; k++) a[row + k] = r[k] ^ (~r[(k + 1) % 5] & r[(k + 2) % 5]);
    }
    a[0] ^= RC[round];
  }
}

class Strobe128 {
 public:
  static constexpr int kRate = 166;
  explicit Strobe128(const uint8_t* label, size_t n) {
    memset(st_, 0, sizeof st_);
    const uint8_t head[6] = {1, kRate + 2, 1, 0, 1, 96};
    memcpy(st_, head, 6);
    memcpy(st_ + 6, "STROBEv1.0.2", 12);
    permute();
    pos_ = pos_begin_ = cur_flags_ = 0;
    meta_ad(label, n, false);
  }
  void meta_ad(const uint8_t* d, size_t n, bool more) { begin_op(kM | kA, more); absorb(d, n); }
  void ad(const uint8_t* d, size_t n, bool more) { begin_op(kA, more); absorb(d, n); }
  void prf(uint8_t* out, size_t n, bool more) { begin_op(kI | kA | kC, more); squeeze(out, n); }

  // raw state access (the device-resident transcript is seeded from / written back to it)
  uint8_t* state() { return st_; }
  uint8_t& pos() { return pos_; }
  uint8_t& pos_begin() { return pos_begin_; }
  uint8_t& cur_flags() { return cur_flags_; }

 private:
  enum : uint8_t { kI = 1, kA = 2, kC = 4, kT = 8, kM = 16, kK = 32 };
  void permute() {
    uint64_t lanes[25];
    memcpy(lanes, st_, 200);  // little-endian host
    keccak_f1600(lanes);
    memcpy(st_, lanes, 200);
  }
  void run_f() {
    st_[pos_] ^= pos_begin_;
    st_[pos_ + 1] ^= 0x04;
    st_[kRate + 1] ^= 0x80;
    permute();
    pos_ = 0;
    pos_begin_ = 0;
  }
  void absorb(const uint8_t* d, size_t n) {
    for (size_t i = 0; i < n; i++) {
      st_[pos_++] ^= d[i];
      if (pos_ == kRate) run_f();
    }
  }
  void squeeze(uint8_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
      out[i] = st_[pos_];
      st_[pos_++] = 0;
      if (pos_ == kRate) run_f();
    }
  }
  void begin_op(uint8_t flags, bool more) {
    if (more) return;  // continuation of the current operation
    const uint8_t old_begin = pos_begin_;
    pos_begin_ = pos_ + 1;
    cur_flags_ = flags;
    const uint8_t hdr[2] = {old_begin, flags};
    absorb(hdr, 2);
    if ((flags & (kC | kK)) && pos_ != 0) run_f();
  }
  uint8_t st_[200];
  uint8_t pos_, pos_begin_, cur_flags_;
};

class MerlinTranscript {
 public:
  MerlinTranscript(const uint8_t* label, size_t n) : strobe_(reinterpret_cast<const uint8_t*>("Merlin v1.0"), 11) {
    append_message(reinterpret_cast<const uint8_t*>("dom-sep"), 7, label, n);
  }
  void append_message(const uint8_t* label, size_t ln, const uint8_t* msg, size_t n) {
    const uint32_t len = (uint32_t)n;
    uint8_t le[4] = {(uint8_t)len, (uint8_t)(len >> 8), (uint8_t)(len >> 16), (uint8_t)(len >> 24)};
    strobe_.meta_ad(label, ln, false);
    strobe_.meta_ad(le, 4, true);
    strobe_.ad(msg, n, false);
  }
  void append_u64(const uint8_t* label, size_t ln, uint64_t v) {
    uint8_t le[8];
    for (int i = 0; i < 8; i++) le[i] = (uint8_t)(v >> (8 * i));
    append_message(label, ln, le, 8);
  }
  void challenge_bytes(const uint8_t* label, size_t ln, uint8_t* out, size_t n) {
    const uint32_t len = (uint32_t)n;
    uint8_t le[4] = {(uint8_t)len, (uint8_t)(len >> 8), (uint8_t)(len >> 16), (uint8_t)(len >> 24)};
    strobe_.meta_ad(label, ln, false);
    strobe_.meta_ad(le, 4, true);
    strobe_.prf(out, n, false);
  }
  Strobe128& strobe() { return strobe_; }

 private:
  Strobe128 strobe_;
};

}  // namespace zk
