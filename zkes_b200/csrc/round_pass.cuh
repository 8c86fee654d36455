// One pass of a dense sumcheck round over this warp's share of the tables: bind the previous
// challenge (FOLD) and accumulate this round's message, shared by the per-round kernel and the
// resident multi-round kernel.
//   fold     u[j]  = t[2j] + r (t[2j+1] - t[2j])                    linear_prover.rs:151-178
//   message  s(c)  = sum_y prod_i (u_i[2y] + c (u_i[2y+1] - u_i[2y])),  c = 0..L   :82-140
#pragma once
#include "internal.hpp"
#include "reduce.cuh"
#include "warp_tile.cuh"

namespace zk {

constexpr int kRoundThreads = 128;
constexpr int kRoundWarps = kRoundThreads / 32;

// src/dst: L tables (dst unused without FOLD); r: multiplier table of the challenge being bound
// (any memory space); pairs: (even, odd) pairs of the table the message is computed over; tiles
// of 32 pairs go to warps warp_global, warp_global + warp_stride, ...; sw: this warp's staging
// tile (WarpTile<8>::kChunks slots).  s[c] receives this thread's share of the message.
// COHERENT: the tables were written earlier in the same launch by other blocks.
template <int L, bool FOLD, bool COHERENT = false, class SrcPtr, class DstPtr>
__device__ __forceinline__ void round_pass(const SrcPtr& src, const DstPtr& dst, const FixedMul<FrParams>& r,
                                           uint64_t pairs, uint64_t warp_global, uint64_t warp_stride, uint4* sw,
                                           int lane, Fr (&s)[L + 1]) {
  const uint64_t tiles = (pairs + 31) >> 5;
  Wide acc[L + 1];
#pragma unroll
  for (int c = 0; c <= L; c++)
#pragma unroll
    for (int k = 0; k < 16; k++) acc[c].v[k] = 0;
  int pending = 0;

  for (uint64_t tile = warp_global; tile < tiles; tile += warp_stride) {
    const uint64_t pair0 = tile << 5;
    const uint32_t valid_pairs = (uint32_t)((pairs - pair0) < 32 ? (pairs - pair0) : 32);
    Fr u0[L], d[L];
    if constexpr (FOLD) {
      uint4 raw[L][8];
#pragma unroll
      for (int i = 0; i < L; i++)
        WarpTile<8>::template issue<COHERENT>(reinterpret_cast<const uint4*>(src[i]) + pair0 * 8, valid_pairs * 8, lane, raw[i]);
#pragma unroll
      for (int i = 0; i < L; i++) {
        uint4 q[8];
        WarpTile<8>::transpose_in(sw, lane, raw[i], q);
        const Fr t0 = fr_from_chunks(q[0], q[1]), t1 = fr_from_chunks(q[2], q[3]);
        const Fr t2 = fr_from_chunks(q[4], q[5]), t3 = fr_from_chunks(q[6], q[7]);
        const Fr a = add(t0, mul_fixed(r, sub(t1, t0)));
        const Fr b = add(t2, mul_fixed(r, sub(t3, t2)));
        uint4 o[4];
        fr_to_chunks(a, o[0], o[1]);
        fr_to_chunks(b, o[2], o[3]);
        WarpTile<4>::store(reinterpret_cast<uint4*>(dst[i]) + pair0 * 4, valid_pairs * 4, sw, lane, o);
        u0[i] = a;
        d[i] = sub(b, a);
      }
    } else {
      uint4 raw[L][4];
#pragma unroll
      for (int i = 0; i < L; i++)
        WarpTile<4>::template issue<COHERENT>(reinterpret_cast<const uint4*>(src[i]) + pair0 * 4, valid_pairs * 4, lane, raw[i]);
#pragma unroll
      for (int i = 0; i < L; i++) {
        uint4 q[4];
        WarpTile<4>::transpose_in(sw, lane, raw[i], q);
        const Fr a = fr_from_chunks(q[0], q[1]), b = fr_from_chunks(q[2], q[3]);
        u0[i] = a;
        d[i] = sub(b, a);
      }
    }
    // lanes past the end of the table hold zeros and add nothing
#pragma unroll
    for (int c = 0; c <= L; c++) {
      Wide w;
      if (L == 1) {
        const Fr one = Fr::one();
        mul_wide(w, u0[0].v, one.v);
      } else {
        Fr prod = u0[0];
#pragma unroll
        for (int i = 1; i < L - 1; i++) prod = mul(prod, u0[i]);
        mul_wide(w, prod.v, u0[L - 1].v);
      }
      wide_add(acc[c], w);
      if (c < L) {
#pragma unroll
        for (int i = 0; i < L; i++) u0[i] = add(u0[i], d[i]);
      }
    }
    if (++pending == kLazyProducts) {
#pragma unroll
      for (int c = 0; c <= L; c++) wide_trim<FrParams>(acc[c]);
      pending = 0;
    }
  }
#pragma unroll
  for (int c = 0; c <= L; c++) {
    wide_trim<FrParams>(acc[c]);
    s[c] = redc<FrParams>(acc[c]);
  }
}

// The same pass with the tiles streamed in by cp.async: while a tile is folded and multiplied, the next one of
// this warp is already on its way into the other stage, so the products do not wait for memory (with 255
// registers a block has few warps to hide that latency otherwise).  stage: this warp's 2 * L tiles of
// WarpTile<8>::kChunks slots; a tile's own slots double as the staging of its folded output.  cp.async.cg reads
// through L2, so tables written earlier in the same launch by other blocks are seen.
template <int L, bool FOLD, class SrcPtr, class DstPtr>
__device__ __forceinline__ void round_pass_async(const SrcPtr& src, const DstPtr& dst, const FixedMul<FrParams>& r,
                                                 uint64_t pairs, uint64_t warp_global, uint64_t warp_stride, uint4* stage,
                                                 int lane, Fr (&s)[L + 1]) {
  constexpr int CH = FOLD ? 8 : 4;
  constexpr int kSlots = WarpTile<8>::kChunks;  // per table and stage, for either variant
  const uint64_t tiles = (pairs + 31) >> 5;
  Wide acc[L + 1];
#pragma unroll
  for (int c = 0; c <= L; c++)
#pragma unroll
    for (int k = 0; k < 16; k++) acc[c].v[k] = 0;
  int pending = 0;
  auto valid_of = [&](uint64_t tile) { return (uint32_t)((pairs - (tile << 5)) < 32 ? (pairs - (tile << 5)) : 32); };
  auto prefetch = [&](uint64_t tile, int buf) {
#pragma unroll
    for (int i = 0; i < L; i++)
      WarpTile<CH>::prefetch_async(stage + (buf * L + i) * kSlots, reinterpret_cast<const uint4*>(src[i]) + (tile << 5) * CH,
                                   valid_of(tile) * CH, lane);
  };
  uint64_t tile = warp_global;
  int buf = 0;
  if (tile < tiles) prefetch(tile, 0);
  for (; tile < tiles; tile += warp_stride, buf ^= 1) {
    const uint64_t pair0 = tile << 5;
    const uint32_t valid_pairs = valid_of(tile);
    const uint64_t next = tile + warp_stride;
    if (next < tiles) {
      prefetch(next, buf ^ 1);
      WarpTile<CH>::template wait_async<L>();  // one commit group per table: the next tile's may stay in flight
    } else {
      WarpTile<CH>::template wait_async<0>();
    }
    Fr u0[L], d[L];
#pragma unroll
    for (int i = 0; i < L; i++) {
      uint4* slots = stage + (buf * L + i) * kSlots;
      uint4 q[CH];
      WarpTile<CH>::read_rows(slots, lane, q);
      if constexpr (FOLD) {
        const Fr t0 = fr_from_chunks(q[0], q[1]), t1 = fr_from_chunks(q[2], q[3]);
        const Fr t2 = fr_from_chunks(q[4], q[5]), t3 = fr_from_chunks(q[6], q[7]);
        const Fr a = add(t0, mul_fixed(r, sub(t1, t0)));
        const Fr b = add(t2, mul_fixed(r, sub(t3, t2)));
        uint4 o[4];
        fr_to_chunks(a, o[0], o[1]);
        fr_to_chunks(b, o[2], o[3]);
        WarpTile<4>::store(reinterpret_cast<uint4*>(dst[i]) + pair0 * 4, valid_pairs * 4, slots, lane, o);
        u0[i] = a;
        d[i] = sub(b, a);
      } else {
        const Fr a = fr_from_chunks(q[0], q[1]), b = fr_from_chunks(q[2], q[3]);
        u0[i] = a;
        d[i] = sub(b, a);
      }
    }
    // lanes past the end of the table hold zeros and add nothing
#pragma unroll
    for (int c = 0; c <= L; c++) {
      Wide w;
      if (L == 1) {
        const Fr one = Fr::one();
        mul_wide(w, u0[0].v, one.v);
      } else {
        Fr prod = u0[0];
#pragma unroll
        for (int i = 1; i < L - 1; i++) prod = mul(prod, u0[i]);
        mul_wide(w, prod.v, u0[L - 1].v);
      }
      wide_add(acc[c], w);
      if (c < L) {
#pragma unroll
        for (int i = 0; i < L; i++) u0[i] = add(u0[i], d[i]);
      }
    }
    if (++pending == kLazyProducts) {
#pragma unroll
      for (int c = 0; c <= L; c++) wide_trim<FrParams>(acc[c]);
      pending = 0;
    }
  }
#pragma unroll
  for (int c = 0; c <= L; c++) {
    wide_trim<FrParams>(acc[c]);
    s[c] = redc<FrParams>(acc[c]);
  }
}

}  // namespace zk
