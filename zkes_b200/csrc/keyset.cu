// Ordering of the entries of SparseBoolSumcheckProver on the device.
//
// The reference sorts every term's position list on the host (linear_prover.rs:497-506).  The entries here
// are 32-bit keys (term << num_var | position), all distinct, in a key space of at most 2^32: they are put
// in order by marking them in a bitmap of the key space and reading the bitmap back in order, which needs
// no comparison sort: one atomic OR per key (its old value exposes a duplicate), a population count per
// 4 KiB block of the bitmap, a scan of the block counts, and an ordered expansion of every block's bits.
#include "internal.hpp"
#include "msm.hpp"

namespace zk {
namespace {

constexpr int kWordsPerBlock = 1024;  // bitmap words (32 keys each) per block of the count / expand passes

// bad[0]: a position >= 2^num_var; bad[1]: the same position twice in one term
__global__ void k_keyset_mark(const uint64_t* __restrict__ positions, const uint64_t* __restrict__ term_begin, uint32_t n_terms,
                              uint64_t total, uint32_t num_var, uint32_t* bitmap, uint32_t* bad) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t lo = 0, hi = n_terms - 1;  // the term whose range [term_begin[t], term_begin[t + 1]) holds i
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo + 1) >> 1);
      if (term_begin[mid] <= i) lo = mid; else hi = mid - 1;
    }
    const uint64_t pos = positions[i];
    if (pos >> num_var) {
      bad[0] = lo + 1;
      continue;
    }
    const uint32_t key = (uint32_t)(((uint64_t)lo << num_var) | pos);
    const uint32_t bit = 1u << (key & 31);
    if (atomicOr(bitmap + (key >> 5), bit) & bit) bad[1] = lo + 1;
  }
}

__global__ void __launch_bounds__(256) k_keyset_count(const uint32_t* __restrict__ bitmap, uint64_t n_words, uint32_t* block_counts) {
  const uint64_t base = (uint64_t)blockIdx.x * kWordsPerBlock;
  int c = 0;
#pragma unroll
  for (int k = 0; k < kWordsPerBlock / 256; k++) {
    const uint64_t w = base + threadIdx.x * (kWordsPerBlock / 256) + k;
    if (w < n_words) c += __popc(bitmap[w]);
  }
  __shared__ int warp_tot[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) c += __shfl_down_sync(0xffffffffu, c, off);
  if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < 8; w++) t += warp_tot[w];
    block_counts[blockIdx.x] = (uint32_t)t;
  }
}

// block_offsets: exclusive scan of the block counts.  Every thread owns four consecutive words; the set
// bits of the block are written in increasing key order.
__global__ void __launch_bounds__(256) k_keyset_expand(const uint32_t* __restrict__ bitmap, uint64_t n_words,
                                                       const uint32_t* __restrict__ block_offsets, uint32_t* keys_out) {
  constexpr int kPer = kWordsPerBlock / 256;
  const uint64_t base = (uint64_t)blockIdx.x * kWordsPerBlock + (uint64_t)threadIdx.x * kPer;
  uint32_t w[kPer];
  uint32_t mine = 0;
#pragma unroll
  for (int k = 0; k < kPer; k++) {
    w[k] = base + k < n_words ? bitmap[base + k] : 0u;
    mine += __popc(w[k]);
  }
  __shared__ uint32_t warp_tot[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t x = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, off);
    if (lane >= off) x += y;
  }
  if (lane == 31) warp_tot[warp] = x;
  __syncthreads();
  uint32_t slot = block_offsets[blockIdx.x] + x - mine;
  for (int v = 0; v < warp; v++) slot += warp_tot[v];
#pragma unroll
  for (int k = 0; k < kPer; k++) {
    uint32_t bits = w[k];
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      keys_out[slot++] = (uint32_t)((base + k) << 5) | (uint32_t)b;
    }
  }
}

}  // namespace

// keys_out[0 .. total) <- the keys (term << num_var | position) in increasing order.  positions_dev: the terms'
// position lists concatenated (device); term_begin_dev: n_terms + 1 prefix offsets (device).  scratch: at least
// keyset_scratch_bytes(...) bytes of device memory.  *bad_host receives {term + 1 with a position out of range or
// 0, term + 1 with a duplicate or 0}.  Synchronises the stream.
size_t keyset_scratch_bytes(uint32_t n_terms, uint32_t num_var) {
  const uint64_t n_words = (((uint64_t)n_terms << num_var) + 31) / 32;
  const uint64_t n_blocks = (n_words + kWordsPerBlock - 1) / kWordsPerBlock;
  return (size_t)(n_words * 4 + 256 + (n_blocks + 2) * 4 + 256 + scan_scratch_elems(n_blocks + 1) * 4 + 512);
}

int keyset_order(zk_ctx* ctx, const uint64_t* positions_dev, const uint64_t* term_begin_dev, uint32_t n_terms, uint64_t total,
                 uint32_t num_var, void* scratch, uint32_t* keys_out, uint32_t bad_host[2]) {
  cudaStream_t s = ctx->stream;
  const uint64_t n_words = (((uint64_t)n_terms << num_var) + 31) / 32;
  const uint64_t n_blocks = (n_words + kWordsPerBlock - 1) / kWordsPerBlock;
  char* p = reinterpret_cast<char*>(scratch);
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(p);
  p += (n_words * 4 + 255) & ~(size_t)255;
  uint32_t* block_counts = reinterpret_cast<uint32_t*>(p);
  p += ((n_blocks + 2) * 4 + 255) & ~(size_t)255;
  uint32_t* scan_tmp = reinterpret_cast<uint32_t*>(p);
  p += (scan_scratch_elems(n_blocks + 1) * 4 + 255) & ~(size_t)255;
  uint32_t* bad = reinterpret_cast<uint32_t*>(p);
  ZK_CUDA(cudaMemsetAsync(bitmap, 0, n_words * 4, s));
  ZK_CUDA(cudaMemsetAsync(bad, 0, 8, s));
  if (total) {
    uint64_t blocks = (total + 255) / 256;
    if (blocks > (uint64_t)ctx->sm_count * 16) blocks = (uint64_t)ctx->sm_count * 16;
    k_keyset_mark<<<(unsigned)blocks, 256, 0, s>>>(positions_dev, term_begin_dev, n_terms, total, num_var, bitmap, bad);
    k_keyset_count<<<(unsigned)n_blocks, 256, 0, s>>>(bitmap, n_words, block_counts);
    ctx->launches += 2 + exclusive_scan_u32(block_counts, n_blocks, scan_tmp, false, s);
    k_keyset_expand<<<(unsigned)n_blocks, 256, 0, s>>>(bitmap, n_words, block_counts, keys_out);
    ctx->launches++;
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, bad, 8, cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  memcpy(bad_host, ctx->host_small, 8);
  return 0;
}

}  // namespace zk
