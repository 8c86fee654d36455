// Multilinear helpers of src/util/poly.rs on the device:
//   eq table   evaluate_lagrange_basis / precompute_eq (poly.rs:573-618, 657-699)
//   fix from right   out[lo] = sum_hi eq[hi] * f[hi * 2^rem + lo]   (poly.rs:705-758)
#include "internal.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

__device__ __forceinline__ Fr ldg_fr(const Fr* p) {
  const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}
__device__ __forceinline__ Fr ld_fr_plain(const Fr* p) {
  const uint4 lo = reinterpret_cast<const uint4*>(p)[0];
  const uint4 hi = reinterpret_cast<const uint4*>(p)[1];
  return fr_from_chunks(lo, hi);
}
__device__ __forceinline__ void st_fr_plain(Fr* p, const Fr& x) {
  uint4 lo, hi;
  fr_to_chunks(x, lo, hi);
  reinterpret_cast<uint4*>(p)[0] = lo;
  reinterpret_cast<uint4*>(p)[1] = hi;
}

// One level of the table: a[x + cur] = r * a[x]; a[x] -= a[x + cur], for x < cur.
__global__ void __launch_bounds__(256) k_eq_level(Fr* a, uint64_t cur, const FixedMul<FrParams> r) {
  for (uint64_t x = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; x < cur; x += (uint64_t)gridDim.x * blockDim.x) {
    const Fr v = ld_fr_plain(a + x);
    const Fr hi = mul_fixed(r, v);
    st_fr_plain(a + x + cur, hi);
    st_fr_plain(a + x, sub(v, hi));
  }
}

// The first levels (table of at most 1024 entries) in one block.
__global__ void __launch_bounds__(512) k_eq_head(Fr* a, const Fr* __restrict__ point, int levels) {
  __shared__ Fr sh[1024];
  if (threadIdx.x == 0) sh[0] = Fr::one();
  __syncthreads();
  for (int i = 0; i < levels; i++) {
    const uint32_t cur = 1u << i;
    const Fr r = point[i];
    if (threadIdx.x < cur) {
      const Fr v = sh[threadIdx.x];
      const Fr hi = mul(r, v);
      sh[threadIdx.x + cur] = hi;
      sh[threadIdx.x] = sub(v, hi);
    }
    __syncthreads();
  }
  for (uint32_t x = threadIdx.x; x < (1u << levels); x += blockDim.x) a[x] = sh[x];
}

// Partial column sums: block (bx, by) covers 256 columns and the hi range of split by.
__global__ void __launch_bounds__(256) k_from_right(const Fr* __restrict__ f, const Fr* __restrict__ eq, uint64_t lo_n,
                                                    uint64_t hi_n, uint64_t hi_per_split, Fr* partial) {
  const uint64_t lo = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (lo >= lo_n) return;
  const uint64_t h0 = (uint64_t)blockIdx.y * hi_per_split;
  const uint64_t h1 = (h0 + hi_per_split < hi_n) ? h0 + hi_per_split : hi_n;
  Wide acc;
#pragma unroll
  for (int k = 0; k < 16; k++) acc.v[k] = 0;
  int pending = 0;
  for (uint64_t h = h0; h < h1; h++) {
    const Fr e = ldg_fr(eq + h);
    const Fr v = ldg_fr(f + h * lo_n + lo);
    Wide w;
    mul_wide(w, v.v, e.v);
    wide_add(acc, w);
    if (++pending == kLazyProducts) {
      wide_trim<FrParams>(acc);
      pending = 0;
    }
  }
  wide_trim<FrParams>(acc);
  st_fr_plain(partial + (uint64_t)blockIdx.y * lo_n + lo, redc<FrParams>(acc));
}

// out[lo] = sum_k partial[k * lo_n + lo].  A block takes 32 columns; its eight warps share the splits (warp g
// sums splits g, g + 8, ...: a warp reads 1 KiB of one split at a time, and the loads of a thread do not wait
// for one another), then the eight partial sums of a column are added through shared memory.
__global__ void __launch_bounds__(256) k_sum_splits(const Fr* __restrict__ partial, uint64_t lo_n, uint32_t splits, Fr* out) {
  __shared__ Fr sh[8][32];
  const int col = threadIdx.x & 31, g = threadIdx.x >> 5;
  const uint64_t lo = (uint64_t)blockIdx.x * 32 + col;
  Fr s = Fr::zero();
  if (lo < lo_n) {
    uint32_t k = g;
    for (; k + 24 < splits; k += 32) {  // four loads in flight
      const Fr a = ld_fr_plain(partial + (uint64_t)k * lo_n + lo), b = ld_fr_plain(partial + (uint64_t)(k + 8) * lo_n + lo);
      const Fr c = ld_fr_plain(partial + (uint64_t)(k + 16) * lo_n + lo), d = ld_fr_plain(partial + (uint64_t)(k + 24) * lo_n + lo);
      s = add(add(s, add(a, b)), add(c, d));
    }
    for (; k < splits; k += 8) s = add(s, ld_fr_plain(partial + (uint64_t)k * lo_n + lo));
  }
  sh[g][col] = s;
  __syncthreads();
  if (g == 0 && lo < lo_n) {
#pragma unroll
    for (int w = 1; w < 8; w++) s = add(s, sh[w][col]);
    st_fr_plain(out + lo, s);
  }
}

// sum_i a[i] * b[i] with lazily reduced products (evaluate_multilinear_extension's final sum, poly.rs:635-647).
__global__ void __launch_bounds__(256) k_dot(const Fr* __restrict__ a, const Fr* __restrict__ b, uint64_t n, const MsgSink sink) {
  Wide acc;
#pragma unroll
  for (int k = 0; k < 16; k++) acc.v[k] = 0;
  int pending = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const Fr x = ldg_fr(a + i), y = ldg_fr(b + i);
    Wide w;
    mul_wide(w, x.v, y.v);
    wide_add(acc, w);
    if (++pending == kLazyProducts) {
      wide_trim<FrParams>(acc);
      pending = 0;
    }
  }
  wide_trim<FrParams>(acc);
  Fr s[1] = {redc<FrParams>(acc)};
  grid_sum<1, 8>(s, sink);
}

}  // namespace

// sink.msg[0] = sum_i a[i] b[i]
void launch_dot(const Fr* a, const Fr* b, uint64_t n, const RoundScratch& sc, cudaStream_t s) {
  uint64_t blocks = (n + 255) / 256;
  const uint64_t cap = (uint64_t)sc.sm_count * 4 < (uint64_t)sc.max_blocks ? sc.sm_count * 4 : sc.max_blocks;
  if (blocks < 1) blocks = 1;
  if (blocks > cap) blocks = cap;
  k_dot<<<(unsigned)blocks, 256, 0, s>>>(a, b, n, sc.sink);
}

// out[0 .. 2^k) = eq(., point); point_dev holds the k coordinates on the device, point_host the
// same values on the host (for the per-level multiplier tables).  Returns launches.
int launch_eq_table(const Fr* point_dev, const Fr* point_host, uint32_t k, Fr* out, int sm_count, cudaStream_t s) {
  const int head = k < 10 ? (int)k : 10;
  k_eq_head<<<1, 512, 0, s>>>(out, point_dev, head);
  int launches = 1;
  for (uint32_t i = head; i < k; i++) {
    const uint64_t cur = 1ull << i;
    uint64_t blocks = (cur + 255) / 256;
    if (blocks > (uint64_t)sm_count * 8) blocks = sm_count * 8;
    k_eq_level<<<(unsigned)blocks, 256, 0, s>>>(out, cur, make_fixed_mul(point_host[i]));
    launches++;
  }
  return launches;
}

uint32_t from_right_splits(uint64_t lo_n, uint64_t hi_n, int sm_count) {
  const uint64_t col_blocks = (lo_n + 255) / 256;
  uint64_t want = ((uint64_t)sm_count * 8 + col_blocks - 1) / col_blocks;  // about 8 blocks per SM
  if (want > hi_n) want = hi_n;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return (uint32_t)want;
}

// out[lo] = sum_hi eq[hi] * f[hi * lo_n + lo]; partial needs from_right_splits() * lo_n elements.
int launch_from_right(const Fr* f, const Fr* eq, uint64_t lo_n, uint64_t hi_n, Fr* partial, Fr* out, int sm_count,
                      cudaStream_t s) {
  const uint32_t splits = from_right_splits(lo_n, hi_n, sm_count);
  const uint64_t per = (hi_n + splits - 1) / splits;
  dim3 grid((unsigned)((lo_n + 255) / 256), splits);
  if (splits == 1) {
    k_from_right<<<grid, 256, 0, s>>>(f, eq, lo_n, hi_n, per, out);
    return 1;
  }
  k_from_right<<<grid, 256, 0, s>>>(f, eq, lo_n, hi_n, per, partial);
  k_sum_splits<<<(unsigned)((lo_n + 31) / 32), 256, 0, s>>>(partial, lo_n, splits, out);
  return 2;
}

}  // namespace zk
