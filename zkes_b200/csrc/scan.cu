// Exclusive prefix sum over u32 arrays of any length (block scan, recursive scan of the block
// totals, uniform add).  Used by the MSM bucket sort.
#include "internal.hpp"

namespace zk {
namespace {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;  // per thread
constexpr uint32_t kScanTile = kScanThreads * kScanItems;

// In place: data[i] <- sum of data[tile start .. i); the tile total goes to sums[blockIdx.x].
__global__ void __launch_bounds__(kScanThreads) k_scan_tile(uint32_t* data, uint64_t n, uint32_t* sums) {
  __shared__ uint32_t warp_tot[kScanThreads / 32];
  const uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint32_t local = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    v[k] = (base + k < n) ? data[base + k] : 0;
    local += v[k];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t x = local;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, off);
    if (lane >= off) x += y;
  }
  if (lane == 31) warp_tot[warp] = x;
  __syncthreads();
  uint32_t before = x - local;
  for (int w = 0; w < warp; w++) before += warp_tot[w];
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    if (base + k < n) data[base + k] = before;
    before += v[k];
  }
  if (threadIdx.x == kScanThreads - 1) sums[blockIdx.x] = before;
}

__global__ void __launch_bounds__(kScanThreads) k_scan_add(uint32_t* data, uint64_t n, const uint32_t* offsets) {
  const uint32_t add = offsets[blockIdx.x];
  const uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
#pragma unroll
  for (int k = 0; k < kScanItems; k++)
    if (base + k < n) data[base + k] += add;
}

}  // namespace

uint64_t scan_scratch_elems(uint64_t n) {
  uint64_t total = 0;
  while (n > 1) {
    n = (n + kScanTile - 1) / kScanTile;
    total += n + 1;
  }
  return total + 2;
}

// data[0..n) <- exclusive prefix sums; the grand total is written to data[n] when
// write_total is set (the caller sizes the array n + 1).  Returns the number of launches.
int exclusive_scan_u32(uint32_t* data, uint64_t n, uint32_t* scratch, bool write_total, cudaStream_t s) {
  if (n == 0) {
    if (write_total) cudaMemsetAsync(data, 0, 4, s);
    return 0;
  }
  const uint64_t tiles = (n + kScanTile - 1) / kScanTile;
  int launches = 1;
  k_scan_tile<<<(unsigned)tiles, kScanThreads, 0, s>>>(data, n, scratch);
  if (tiles > 1) {
    // scratch[0..tiles) holds tile totals; scan them in place (total lands in scratch[tiles])
    launches += exclusive_scan_u32(scratch, tiles, scratch + tiles + 1, true, s);
    k_scan_add<<<(unsigned)tiles, kScanThreads, 0, s>>>(data, n, scratch);
    launches++;
    if (write_total) cudaMemcpyAsync(data + n, scratch + tiles, 4, cudaMemcpyDeviceToDevice, s);
  } else if (write_total) {
    cudaMemcpyAsync(data + n, scratch, 4, cudaMemcpyDeviceToDevice, s);
  }
  return launches;
}

}  // namespace zk
