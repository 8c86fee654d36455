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

  // Coalesced global reads into registers; chunks at or beyond `valid` read as zero.  COHERENT
  // reads through L2 only (ld.cg): for data that other blocks of the same launch have written.
  template <bool COHERENT = false>
  static __device__ __forceinline__ void issue(const uint4* __restrict__ g, uint32_t valid, int lane,
                                               uint4 (&raw)[CH]) {
#pragma unroll
    for (int j = 0; j < CH; j++) {
      const uint32_t c = j * 32 + lane;
      raw[j] = (c < valid) ? (COHERENT ? __ldcg(g + c) : __ldg(g + c)) : make_uint4(0, 0, 0, 0);
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

  // Asynchronous form of issue + the first half of transpose_in: the tile goes from global memory
  // straight into its swizzled shared-memory slots (16-byte cp.async, no registers), as one commit
  // group.  Chunks at or beyond `valid` are zero-filled.  Pair with wait_async + read_rows.
  static __device__ __forceinline__ void prefetch_async(uint4* smem_warp, const uint4* __restrict__ g, uint32_t valid,
                                                        int lane) {
#pragma unroll
    for (int j = 0; j < CH; j++) {
      const uint32_t c = j * 32 + lane;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_warp + phys(c / CH, c % CH));
      const uint32_t bytes = c < valid ? 16u : 0u;  // 0: nothing is read, the slot is zero-filled
      const uint4* src = c < valid ? g + c : g;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  // Wait until at most `Pending` of this thread's commit groups are still in flight, then make the
  // warp's copies visible to all its lanes.
  template <int Pending>
  static __device__ __forceinline__ void wait_async() {
    asm volatile("cp.async.wait_group %0;" ::"n"(Pending) : "memory");
    __syncwarp();
  }

  static __device__ __forceinline__ void read_rows(const uint4* smem_warp, int lane, uint4 (&out)[CH]) {
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
