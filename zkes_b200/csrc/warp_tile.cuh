// Warp-cooperative staging of contiguous global memory through shared memory.
//
// A lane that needs CH consecutive 16-byte chunks (CH*16 bytes: one to four field elements)
// would touch one cache line per lane with its own loads.  Instead the warp reads the whole
// tile of 32*CH chunks with CH fully coalesced 128-bit loads per lane, parks it in a
// swizzled shared-memory tile and each lane picks up its own row.  Stores go the other way.
// The swizzle (column ^ row-group) makes both phases bank-conflict free for CH = 2, 4, 8.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace zk {

template <int CH>
struct WarpTile {
  static_assert(CH == 2 || CH == 4 || CH == 8, "tile rows are 32, 64 or 128 bytes");
  static constexpr int kChunks = 32 * CH;  // uint4 slots of shared memory per warp

  static __device__ __forceinline__ int phys(int row, int col) {
    return row * CH + (col ^ ((row / (8 / CH)) % CH));
  }

  // Coalesced global reads into registers; chunks at or beyond `valid` read as zero.
  static __device__ __forceinline__ void issue(const uint4* __restrict__ g, uint32_t valid, int lane,
                                               uint4 (&raw)[CH]) {
#pragma unroll
    for (int j = 0; j < CH; j++) {
      const uint32_t c = j * 32 + lane;
      raw[j] = (c < valid) ? __ldg(g + c) : make_uint4(0, 0, 0, 0);
    }
  }

  // raw (coalesced order) -> shared -> out (lane's own CH consecutive chunks).
  static __device__ __forceinline__ void transpose_in(uint4* smem_warp, int lane, const uint4 (&raw)[CH],
                                                      uint4 (&out)[CH]) {
#pragma unroll
    for (int j = 0; j < CH; j++) {
      const int c = j * 32 + lane;
      smem_warp[phys(c / CH, c % CH)] = raw[j];
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < CH; k++) out[k] = smem_warp[phys(lane, k)];
    __syncwarp();
  }

  // Lane's own CH chunks -> shared -> coalesced global writes (chunks below `valid` only).
  static __device__ __forceinline__ void store(uint4* __restrict__ g, uint32_t valid, uint4* smem_warp, int lane,
                                               const uint4 (&in)[CH]) {
#pragma unroll
    for (int k = 0; k < CH; k++) smem_warp[phys(lane, k)] = in[k];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < CH; j++) {
      const uint32_t c = j * 32 + lane;
      if (c < valid) g[c] = smem_warp[phys(c / CH, c % CH)];
    }
    __syncwarp();
  }
};

}  // namespace zk
