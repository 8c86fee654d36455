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

// A field element handed from one block to another without a fence or a separate flag: three 16-byte chunks, each
// written and read as one transaction and each carrying the tag of the hand-over in its last word.  The reader polls
// the chunks until all three show the tag it expects.
struct alignas(16) TaggedFr {
  uint32_t w[3][4];  // {v0, v1, v2, tag}, {v3, v4, v5, tag}, {v6, v7, 0, tag}
  uint32_t pad[4];
};

// Hand-over area of the resident multi-round kernel (device global memory).
struct ResidentShared {
  unsigned int arrive;       // blocks that have added their share of a message, counted up over all rounds in step
  unsigned int seq;          // (unused)
  unsigned int error;        // non-zero: a bounded wait ran out
  unsigned int garrive;      // block tickets of the grid sums (rounds whose message is prepared ahead)
  unsigned int gseq;         // grid of message `gseq - 1` is complete in gsum[(gseq - 1) & 1]
  unsigned int pad[3];
  TaggedFr rplain[2];        // the challenge of round t as a canonical integer in rplain[t & 1], tag t + 1
  TaggedFr gsum[2][16];      // message t tabulated as a polynomial in the challenge before it, scaled, in gsum[t & 1], tag t + 1
  unsigned long long gacc[2][16][8];  // the same grid while the blocks add their shares: 64-bit sums of 32-bit limbs
  unsigned long long macc[2][5][8];   // rounds in step: message t while the blocks add their shares, in macc[t & 1]
  // What a launch that stops before the end of the protocol leaves for the kernel that goes on; not cleared by
  // the next launch, which may be that kernel.
  Fr challenge;              // the last challenge (Montgomery form), still to be bound on the tables
  StrobeState st;            // transcript state after that challenge
};
constexpr int kResidentGrid = 16;  // grid points of a message: (L + 1)^2 for L <= 3

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

#ifdef __CUDACC__
// ---- warp-parallel form: state lane i lives in thread i of one warp (threads 25..31 idle along).
// Every function below is collective over the full warp.

static __constant__ uint64_t kKeccakRcDev[24] = {
    0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808Aull, 0x8000000080008000ull,
    0x000000000000808Bull, 0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull,
    0x000000000000008Aull, 0x0000000000000088ull, 0x0000000080008009ull, 0x000000008000000Aull,
    0x000000008000808Bull, 0x800000000000008Bull, 0x8000000000008089ull, 0x8000000000008003ull,
    0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800Aull, 0x800000008000000Aull,
    0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};

// One Keccak-f[1600] over a warp, exchanging lanes through shared memory: a 64-bit load moves a
// whole lane where a shuffle moves half of one, and a 128-bit load two.  Per round: every thread
// parks its lane column-major, reads its two neighbour columns (theta, 6 loads), rotates (rho),
// parks the result at its pi position row-major and reads the three lanes of its row that chi
// needs.  scratch: 2 x 32 eight-byte slots, 16-byte aligned, private to the warp.
static __device__ __noinline__ uint2 keccak_f1600_warp(uint2 a, int lane, uint64_t* scratch) {
  const int l = lane < 25 ? lane : 0;  // idle threads mirror lane 0's indices; they store nothing
  const int x = l % 5, y = l / 5;
  // rho offsets, lane = x + 5 y, packed 6 bits each
  const int my_rot = (int)((l < 10 ? (0x5371AC91B73E040ull >> (6 * l))                     // 0 1 62 28 27 36 44 6 55 20
                                   : l < 20 ? (0x2153EDA6766B283ull >> (6 * (l - 10)))      // 3 10 43 25 39 41 45 15 21 8
                                            : (0xEE3D092ull >> (6 * (l - 20)))) & 63);      // 18 2 61 56 14
  const bool swap_halves = my_rot >= 32;
  const int sh = my_rot & 31;
  // column-major tile A (column stride 6 slots) and row-major tile B (row stride 6 slots)
  uint64_t* A = scratch;
  uint64_t* B = scratch + 32;
  uint64_t* a_slot = A + 6 * x + y;
  const uint64_t* col_p = A + 6 * ((x + 4) % 5);
  const uint64_t* col_n = A + 6 * ((x + 1) % 5);
  // pi: lane (x, y) moves to (y, (2x + 3y) mod 5)
  uint64_t* b_slot = B + 6 * ((2 * x + 3 * y) % 5) + y;
  const uint64_t* row = B + 6 * y;
  const int x1 = (x + 1) % 5, x2 = (x + 2) % 5;
  uint32_t lo = a.x, hi = a.y;
#pragma unroll
  for (int round = 0; round < 24; round++) {
    const uint64_t rc = kKeccakRcDev[round];  // uniform load; selected, not branched on, so the warp stays converged
    if (lane < 25) *reinterpret_cast<uint2*>(a_slot) = make_uint2(lo, hi);
    __syncwarp();
    const uint4 p01 = *reinterpret_cast<const uint4*>(col_p), p23 = *reinterpret_cast<const uint4*>(col_p + 2);
    const uint2 p4 = *reinterpret_cast<const uint2*>(col_p + 4);
    const uint4 n01 = *reinterpret_cast<const uint4*>(col_n), n23 = *reinterpret_cast<const uint4*>(col_n + 2);
    const uint2 n4 = *reinterpret_cast<const uint2*>(col_n + 4);
    const uint32_t plo = p01.x ^ p01.z ^ p23.x ^ p23.z ^ p4.x, phi = p01.y ^ p01.w ^ p23.y ^ p23.w ^ p4.y;
    const uint32_t nlo = n01.x ^ n01.z ^ n23.x ^ n23.z ^ n4.x, nhi = n01.y ^ n01.w ^ n23.y ^ n23.w ^ n4.y;
    lo ^= plo ^ __funnelshift_l(nhi, nlo, 1);
    hi ^= phi ^ __funnelshift_l(nlo, nhi, 1);
    const uint32_t tl = swap_halves ? hi : lo, th = swap_halves ? lo : hi;
    const uint32_t rlo = __funnelshift_l(th, tl, sh), rhi = __funnelshift_l(tl, th, sh);
    if (lane < 25) *reinterpret_cast<uint2*>(b_slot) = make_uint2(rlo, rhi);
    __syncwarp();
    const uint2 b0 = *reinterpret_cast<const uint2*>(row + x), b1 = *reinterpret_cast<const uint2*>(row + x1),
                b2 = *reinterpret_cast<const uint2*>(row + x2);
    lo = b0.x ^ (~b1.x & b2.x) ^ (lane == 0 ? (uint32_t)rc : 0u);
    hi = b0.y ^ (~b1.y & b2.y) ^ (lane == 0 ? (uint32_t)(rc >> 32) : 0u);
  }
  return make_uint2(lo, hi);
}

struct WarpStrobe {
  uint64_t a;                // this thread's state lane (threads 0..24)
  uint32_t pos, pos_begin;   // identical in every thread
  uint64_t* scratch;         // 64 eight-byte slots of shared memory (16-byte aligned) for the permutation

  __device__ __forceinline__ void run_f(int lane) {
    if ((int)(pos >> 3) == lane) a ^= (uint64_t)(pos_begin & 0xffu) << (8 * (pos & 7));
    if ((int)((pos + 1) >> 3) == lane) a ^= (uint64_t)0x04 << (8 * ((pos + 1) & 7));
    if (lane == 20) a ^= (uint64_t)0x80 << 56;  // byte kStrobeRate + 1 = 167
    __syncwarp();  // shuffles between diverged threads are far slower than between converged ones
    const uint2 t = keccak_f1600_warp(make_uint2((uint32_t)a, (uint32_t)(a >> 32)), lane, scratch);
    a = ((uint64_t)t.y << 32) | t.x;
    pos = 0;
    pos_begin = 0;
  }
  // XOR m bytes of buf (shared memory, visible to the warp) into the state from byte `start`.
  __device__ __forceinline__ void xor_segment(const uint8_t* buf, uint32_t start, uint32_t m, int lane) {
#pragma unroll
    for (int b = 0; b < 8; b++) {
      const uint32_t p = 8u * lane + b;
      if (lane < 25 && p >= start && p < start + m) a ^= (uint64_t)buf[p - start] << (8 * b);
    }
    __syncwarp();
  }

  // Bytes of one sumcheck round as the transcript sees them (transcript.rs:27-42 over Merlin's framing):
  // per evaluation [begin, 0x12] "round_message" len32 [begin, 0x02] 32 data bytes, then
  // [begin, 0x12] "challenge" len64 [begin, 0x07].  The `begin` bytes depend on the position and are
  // filled in while absorbing; everything else but the data is constant.
  template <int L>
  static constexpr int round_stream_bytes() { return 53 * (L + 1) + 17; }

  template <int L>
  static __device__ void init_round_stream(uint8_t* stream) {  // one thread
    const char* l1 = "round_message";
    const char* l2 = "challenge";
    for (int c = 0; c <= L; c++) {
      uint8_t* s = stream + 53 * c;
      s[0] = 0; s[1] = 16u | 2u;
      for (int i = 0; i < 13; i++) s[2 + i] = (uint8_t)l1[i];
      s[15] = 32; s[16] = 0; s[17] = 0; s[18] = 0;
      s[19] = 0; s[20] = 2u;
    }
    uint8_t* s = stream + 53 * (L + 1);
    s[0] = 0; s[1] = 16u | 2u;
    for (int i = 0; i < 9; i++) s[2 + i] = (uint8_t)l2[i];
    s[11] = 64; s[12] = 0; s[13] = 0; s[14] = 0;
    s[15] = 0; s[16] = 1u | 2u | 4u;
  }
  static __device__ __forceinline__ uint8_t* round_stream_data(uint8_t* stream, int c) { return stream + 53 * c + 21; }

  // Absorbs the round's stream (data bytes already written, warp synchronised), draws the 64
  // challenge bytes and returns the first 32 as eight little-endian words in every thread.
  template <int L>
  __device__ __forceinline__ void fs_round(uint8_t* stream, int lane, uint32_t* raw) {
    constexpr int kPieces = 2 * (L + 1) + 2;
    uint32_t off = 0, seg_off = 0, seg_pos = pos;
#pragma unroll 1
    for (int j = 0; j < kPieces; j++) {
      const uint32_t len = j == kPieces - 1 ? 0u : (j == kPieces - 2 ? 13u : ((j & 1) ? 32u : 17u));
      if (lane == 0) stream[off] = (uint8_t)pos_begin;  // the operation's first framing byte
      pos_begin = pos + 1;
      uint32_t n = 2 + len;
      while (pos + n >= kStrobeRate) {  // the block fills up inside this piece
        const uint32_t take = kStrobeRate - pos;
        __syncwarp();
        xor_segment(stream + seg_off, seg_pos, off + take - seg_off, lane);
        pos = kStrobeRate;
        run_f(lane);
        off += take;
        n -= take;
        seg_off = off;
        seg_pos = 0;
      }
      pos += n;
      off += n;
    }
    __syncwarp();
    xor_segment(stream + seg_off, seg_pos, off - seg_off, lane);
    if (pos != 0) run_f(lane);  // the PRF operation starts on a fresh block
    // squeeze: the 64 bytes at position 0 are state lanes 0..7; they are zeroed behind the read
    const uint32_t lo = (uint32_t)a, hi = (uint32_t)(a >> 32);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      raw[2 * i] = __shfl_sync(0xffffffffu, lo, i);
      raw[2 * i + 1] = __shfl_sync(0xffffffffu, hi, i);
    }
    if (lane < 8) a = 0;
    pos = 64;
    __syncwarp();
  }
};
#endif  // __CUDACC__

}  // namespace zk
