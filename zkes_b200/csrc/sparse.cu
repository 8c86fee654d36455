// Sparse x dense product sumcheck: sum_x a(x) b(x) with a given by K sorted non-zero entries.
//
// While the live domain is much larger than K the prover keeps `a` as (index, value) entries:
// the round message only needs b at the entries' pair positions, the dense table b is folded
// by the plain fold kernel, and the entries are folded by a merge of adjacent indices followed
// by a stream compaction.  Once the domain has shrunk to about the entry count the entries are
// scattered into a dense table and the dense round kernel takes over.  The outputs equal those
// of the dense prover on [a.to_dense(), b] (linear_prover.rs:43-191): zero entries of `a`
// contribute nothing to any message.
#include <cstring>
#include "internal.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

constexpr int kSpThreads = 256;

__device__ __forceinline__ Fr ld_fr(const Fr* p) {
  const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}
__device__ __forceinline__ void st_fr(Fr* p, const Fr& x) {
  uint4 lo, hi;
  fr_to_chunks(x, lo, hi);
  reinterpret_cast<uint4*>(p)[0] = lo;
  reinterpret_cast<uint4*>(p)[1] = hi;
}

// An entry leads its pair unless it is the odd partner of the entry just before it.
__device__ __forceinline__ bool is_leader(const uint32_t* idx, uint32_t i, uint32_t pos) {
  return (pos & 1u) == 0 || i == 0 || idx[i - 1] != pos - 1;
}

// With DEFERRED the dense table has not been folded by the previous challenge yet: the two
// values an entry pair needs are folded on the fly from four consecutive entries.
//
// The message is additive over the entries: with (b0, b1) the dense pair at an entry's pair position,
//   s(0) = sum over even entries v b0,   s(1) = sum over odd entries v b1,
//   s(2) = sum_y (2 v1 - v0)(2 b1 - b0) = sum over even entries v (b0 - 2 b1) + sum over odd entries v (4 b1 - 2 b0),
// so an entry never looks at its neighbour and costs two products whatever its parity: v times the dense value
// on its own side (added to s(0) or s(1) by a mask, so that the warp does not branch on the parity) and v times
// e = b0 - 2 b1 or -2 e.
//
// The fold of the entries is additive in the same way: binding r on a table sends an even entry (pos, v) to
// (pos / 2, (1 - r) v) and an odd one to (pos / 2, r v).  Two entries that land on one position are simply both
// kept (the list stays sorted, and every sum above is linear in v), so the entries are never merged or
// compacted while the prover is in entry form; with FOLD the kernel binds the previous round's challenge on
// its entries first and writes them back in place, which makes one launch per round.
//
// The gather of the dense values depends on the entry's position, and a thread has few entries: without care
// the kernel waits on that chain.  Every thread therefore runs a two-stage pipeline of asynchronous copies into
// its own shared-memory slots (no registers held): while entry k is computed, the dense values and the value of
// entry k + 1 are in flight and the position of entry k + 2 is being loaded.
template <bool DEFERRED, bool FOLD>
__global__ void __launch_bounds__(kSpThreads, 2) k_sparse_msg(uint32_t* __restrict__ idx, Fr* __restrict__ val,
                                                              const uint32_t* __restrict__ count,
                                                              const Fr* __restrict__ dense, const FixedMul<FrParams> pend,
                                                              const FixedMul<FrParams> bind, const MsgSink sink,
                                                              const PeerExchange px, const unsigned int xseq) {
  constexpr int DCH = DEFERRED ? 8 : 4;  // 16-byte chunks of dense values per entry
  constexpr int CH = DCH + 2;            // plus the entry's value
  extern __shared__ uint4 sp_stage[];    // [2 slots][CH chunks][kSpThreads]: a thread's chunks are kSpThreads apart
  const uint32_t n = *count;
  const uint32_t stride = gridDim.x * blockDim.x;
  const int tid = threadIdx.x;
  auto issue = [&](int slot, uint32_t e, uint32_t stored_pos) {
    const uint32_t pos = FOLD ? stored_pos >> 1 : stored_pos;
    const uint4* src = reinterpret_cast<const uint4*>(dense + (DEFERRED ? 4 * (uint64_t)(pos >> 1) : (uint64_t)(pos & ~1u)));
    const uint4* vsrc = reinterpret_cast<const uint4*>(val + e);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sp_stage + ((size_t)(slot * CH + c) * kSpThreads + tid));
      const uint4* g = c < DCH ? src + c : vsrc + (c - DCH);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(g) : "memory");
    }
  };
  auto staged = [&](int slot, int c) { return sp_stage[(size_t)(slot * CH + c) * kSpThreads + tid]; };
  Wide acc[3];
#pragma unroll
  for (int c = 0; c < 3; c++)
#pragma unroll
    for (int k = 0; k < 16; k++) acc[c].v[k] = 0;
  int pending = 0;
  uint32_t i = blockIdx.x * blockDim.x + tid, inext = i + stride;
  uint32_t st_cur = i < n ? idx[i] : 0u, st_next = inext < n ? idx[inext] : 0u;
  if (i < n) issue(0, i, st_cur);
  asm volatile("cp.async.commit_group;" ::: "memory");
  int slot = 0;
  while (i < n) {
    if (inext < n) issue(slot ^ 1, inext, st_next);
    asm volatile("cp.async.commit_group;" ::: "memory");  // one group per iteration, empty or not
    const uint32_t inn = inext < n ? inext + stride : inext;  // (no wrap: inext >= n stays put)
    const uint32_t st_nn = inn < n ? idx[inn] : 0u;
    asm volatile("cp.async.wait_group 1;" ::: "memory");    // the copies of entry i have landed
    uint32_t pos = st_cur;
    Fr v = fr_from_chunks(staged(slot, DCH), staged(slot, DCH + 1));
    if (FOLD) {
      const Fr t = mul_fixed(bind, v);  // r v
      v = (pos & 1u) ? t : sub(v, t);
      pos >>= 1;
      idx[i] = pos;
      st_fr(val + i, v);
    }
    const bool odd = (pos & 1u) != 0;
    Fr b0, b1;
    if (DEFERRED) {
      const Fr t0 = fr_from_chunks(staged(slot, 0), staged(slot, 1)), t1 = fr_from_chunks(staged(slot, 2), staged(slot, 3));
      const Fr t2 = fr_from_chunks(staged(slot, 4), staged(slot, 5)), t3 = fr_from_chunks(staged(slot, 6), staged(slot, 7));
      b0 = add(t0, mul_fixed(pend, sub(t1, t0)));
      b1 = add(t2, mul_fixed(pend, sub(t3, t2)));
    } else {
      b0 = fr_from_chunks(staged(slot, 0), staged(slot, 1));
      b1 = fr_from_chunks(staged(slot, 2), staged(slot, 3));
    }
    const Fr e = sub(b0, dbl(b1));
    const Fr e_odd = neg(dbl(e));
    Fr side, two;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      side.v[k] = odd ? b1.v[k] : b0.v[k];
      two.v[k] = odd ? e_odd.v[k] : e.v[k];
    }
    Wide w;
    mul_wide(w, v.v, side.v);
    const uint32_t m1 = odd ? 0xffffffffu : 0u, m0 = ~m1;
    Wide w0, w1;
#pragma unroll
    for (int k = 0; k < 16; k++) {
      w0.v[k] = w.v[k] & m0;
      w1.v[k] = w.v[k] & m1;
    }
    wide_add(acc[0], w0);
    wide_add(acc[1], w1);
    mul_wide(w, v.v, two.v);
    wide_add(acc[2], w);
    if (++pending == kLazyProducts) {
#pragma unroll
      for (int c = 0; c < 3; c++) wide_trim<FrParams>(acc[c]);
      pending = 0;
    }
    i = inext;
    inext = inn;
    st_cur = st_next;
    st_next = st_nn;
    slot ^= 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  Fr s[3];
#pragma unroll
  for (int c = 0; c < 3; c++) {
    wide_trim<FrParams>(acc[c]);
    s[c] = redc<FrParams>(acc[c]);
  }
  if (xseq)  // one rank of a sharded instance: the last block exchanges the message with the other ranks' kernels
    grid_sum_exchange<3, kSpThreads / 32>(s, sink, px, xseq);
  else
    grid_sum<3, kSpThreads / 32>(s, sink);
}

// Pass 1 of the entry fold: leaders per block.
__global__ void __launch_bounds__(kSpThreads) k_sparse_count(const uint32_t* __restrict__ idx,
                                                             const uint32_t* __restrict__ count,
                                                             uint32_t* block_counts) {
  const uint32_t n = *count;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool lead = i < n && is_leader(idx, i, idx[i]);
  const int c = __syncthreads_count(lead);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = (uint32_t)c;
}

// Pass 2: exclusive scan of the block counts by one block; total goes to count_out.  Eight counts per thread and
// sweep (a serial prefix inside the thread, then the usual two-level scan of the thread totals), so that the half
// million counts of a 2^27-entry list take sixty sweeps.
constexpr int kScanPerThread = 8;
__global__ void __launch_bounds__(1024) k_scan_blocks(uint32_t* block_counts, uint32_t n_blocks, uint32_t* count_out) {
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t base = 0; base < n_blocks; base += 1024 * kScanPerThread) {
    const uint32_t i0 = base + threadIdx.x * kScanPerThread;
    uint32_t c[kScanPerThread];
    uint32_t v = 0;
#pragma unroll
    for (int k = 0; k < kScanPerThread; k++) {
      c[k] = i0 + k < n_blocks ? block_counts[i0 + k] : 0;
      v += c[k];
    }
    uint32_t x = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, x, off);
      if (lane >= off) x += y;
    }
    if (lane == 31) warp_tot[warp] = x;
    __syncthreads();
    if (warp == 0) {
      uint32_t t = warp_tot[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, t, off);
        if (lane >= off) t += y;
      }
      warp_tot[lane] = t;  // inclusive over warps
    }
    __syncthreads();
    uint32_t before = carry + (warp ? warp_tot[warp - 1] : 0) + x - v;
    const uint32_t sweep_total = warp_tot[31];
#pragma unroll
    for (int k = 0; k < kScanPerThread; k++) {
      if (i0 + k < n_blocks) block_counts[i0 + k] = before;
      before += c[k];
    }
    __syncthreads();
    if (threadIdx.x == 0) carry += sweep_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) *count_out = carry;
}

// Pass 3: fold each pair and write it at its compacted slot.
__global__ void __launch_bounds__(kSpThreads) k_sparse_fold(const uint32_t* __restrict__ idx, const Fr* __restrict__ val,
                                                            const uint32_t* __restrict__ count,
                                                            const uint32_t* __restrict__ block_offsets,
                                                            const FixedMul<FrParams> r,
                                                            uint32_t* idx_out, Fr* val_out) {
  __shared__ uint32_t warp_cnt[kSpThreads / 32];
  const uint32_t n = *count;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t pos = 0;
  bool lead = false;
  if (i < n) {
    pos = idx[i];
    lead = is_leader(idx, i, pos);
  }
  const unsigned int ballot = __ballot_sync(0xffffffffu, lead);
  if (lane == 0) warp_cnt[warp] = __popc(ballot);
  __syncthreads();
  if (!lead) return;
  uint32_t slot = block_offsets[blockIdx.x] + __popc(ballot & ((1u << lane) - 1u));
  for (int w = 0; w < warp; w++) slot += warp_cnt[w];
  Fr v0 = Fr::zero(), v1 = Fr::zero();
  if ((pos & 1u) == 0) {
    v0 = ld_fr(val + i);
    if (i + 1 < n && idx[i + 1] == pos + 1) v1 = ld_fr(val + i + 1);
  } else {
    v1 = ld_fr(val + i);
  }
  idx_out[slot] = pos >> 1;
  st_fr(val_out + slot, add(v0, mul_fixed(r, sub(v1, v0))));
}

__global__ void k_scatter(const uint32_t* __restrict__ idx, const Fr* __restrict__ val,
                          const uint32_t* __restrict__ count, Fr* dense) {
  const uint32_t n = *count;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    st_fr(dense + idx[i], ld_fr(val + i));
}

// Entries bound by r in place (the step k_sparse_msg<., true> does on the fly), for the hand-over to the dense form.
__global__ void k_sparse_bind(uint32_t* __restrict__ idx, Fr* __restrict__ val, const uint32_t* __restrict__ count,
                              const FixedMul<FrParams> bind) {
  const uint32_t n = *count;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint32_t pos = idx[i];
    const Fr v = ld_fr(val + i);
    const Fr t = mul_fixed(bind, v);
    idx[i] = pos >> 1;
    st_fr(val + i, (pos & 1u) ? t : sub(v, t));
  }
}

// Dense table from a sorted entry list that may hold several entries per position: the first entry of a run adds
// up its run (a run is at most 2^rounds long and short in practice) and writes the position.
__global__ void k_scatter_runs(const uint32_t* __restrict__ idx, const Fr* __restrict__ val,
                               const uint32_t* __restrict__ count, Fr* dense) {
  const uint32_t n = *count;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint32_t pos = idx[i];
    if (i && idx[i - 1] == pos) continue;
    Fr s = ld_fr(val + i);
    for (uint32_t j = i + 1; j < n && idx[j] == pos; j++) s = add(s, ld_fr(val + j));
    st_fr(dense + pos, s);
  }
}

// 1 when idx[0..n) is strictly increasing and below `limit`, else 0.
__global__ void k_check_sorted(const uint32_t* __restrict__ idx, uint32_t n, uint64_t limit, uint32_t* bad) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if ((uint64_t)idx[i] >= limit || (i > 0 && idx[i - 1] >= idx[i])) *bad = 1;
  }
}

// Flags any idx[i] >= limit.
__global__ void k_check_bound(const uint32_t* __restrict__ idx, uint32_t n, uint64_t limit, uint32_t* bad) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    if ((uint64_t)idx[i] >= limit) *bad = 1;
}

// Narrow caller indices (u64) to the 32-bit form the kernels use; flags values >= 2^32.
// With clamp_below > 0 a value at or above it is flagged and stored as clamp_below - 1, so that the kernels after
// this one stay inside their tables whatever the caller passed (the host looks at the flag later).
__global__ void k_narrow_idx(const uint64_t* __restrict__ in, uint32_t n, uint32_t* out, uint32_t* bad, uint64_t clamp_below) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    uint64_t v = in[i];
    if (v >> 32) *bad = 1;
    if (clamp_below && v >= clamp_below) {
      *bad = 1;
      v = clamp_below - 1;
    }
    out[i] = (uint32_t)v;
  }
}

// Final values when the prover ended in entry form: a = entry 0 if its index is 0, else 0.
__global__ void k_sd_final(const uint32_t* idx, const Fr* val, const uint32_t* count, const Fr* dense, Fr* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  Fr a = Fr::zero();
  if (*count > 0 && idx[0] == 0) a = val[0];
  const Fr b = dense[0];
  out[0] = a;
  out[1] = b;
  out[2] = mul(a, b);
}

inline int blocks_for(uint64_t n, int threads, int cap) {
  uint64_t b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > (uint64_t)cap) b = cap;
  return (int)b;
}

}  // namespace

// pending: the challenge the dense table still has to be folded by, or nullptr.  bind: the challenge the entries
// still have to be bound on (done first, in place), or nullptr.
template <bool D, bool F>
static void launch_sparse_msg_t(uint32_t* idx, Fr* val, const uint32_t* count, uint32_t upper, const Fr* dense,
                                const FixedMul<FrParams>& pt, const FixedMul<FrParams>& bt, const RoundScratch& sc,
                                cudaStream_t s, const PeerExchange& px, unsigned int xseq) {
  constexpr size_t smem = (size_t)2 * ((D ? 8 : 4) + 2) * kSpThreads * sizeof(uint4);
  cudaFuncSetAttribute(k_sparse_msg<D, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_sparse_msg<D, F>, kSpThreads, smem) != cudaSuccess || occ < 1) occ = 1;
  // one wave of resident blocks: every thread walks its entries through the copy pipeline
  int cap = sc.sm_count * occ;
  if (cap > sc.max_blocks) cap = sc.max_blocks;
  const int grid = blocks_for(upper, kSpThreads, cap);
  k_sparse_msg<D, F><<<grid, kSpThreads, smem, s>>>(idx, val, count, dense, pt, bt, sc.sink, px, xseq);
}

void launch_sparse_msg(uint32_t* idx, Fr* val, const uint32_t* count, uint32_t upper, const Fr* dense,
                       const Fr* pending, const Fr* bind, const RoundScratch& sc, cudaStream_t s, const PeerExchange* exchange,
                       unsigned int xseq) {
  PeerExchange px;
  if (exchange) {
    px = *exchange;
  } else {
    memset(&px, 0, sizeof px);
    xseq = 0;
  }
  const FixedMul<FrParams> pt = pending ? make_fixed_mul(*pending) : FixedMul<FrParams>();
  const FixedMul<FrParams> bt = bind ? make_fixed_mul(*bind) : FixedMul<FrParams>();
  if (pending && bind)
    launch_sparse_msg_t<true, true>(idx, val, count, upper, dense, pt, bt, sc, s, px, xseq);
  else if (pending)
    launch_sparse_msg_t<true, false>(idx, val, count, upper, dense, pt, bt, sc, s, px, xseq);
  else if (bind)
    launch_sparse_msg_t<false, true>(idx, val, count, upper, dense, pt, bt, sc, s, px, xseq);
  else
    launch_sparse_msg_t<false, false>(idx, val, count, upper, dense, pt, bt, sc, s, px, xseq);
}

void launch_sparse_bind(uint32_t* idx, Fr* val, const uint32_t* count, uint32_t upper, const Fr& r, int sm_count,
                        cudaStream_t s) {
  k_sparse_bind<<<blocks_for(upper, 256, sm_count * 8), 256, 0, s>>>(idx, val, count, make_fixed_mul(r));
}

void launch_scatter_runs(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, Fr* dense,
                         int sm_count, cudaStream_t s) {
  k_scatter_runs<<<blocks_for(upper, 256, sm_count * 8), 256, 0, s>>>(idx, val, count, dense);
}

int launch_sparse_fold(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, const Fr& r,
                       uint32_t* block_counts, uint32_t* idx_out, Fr* val_out, uint32_t* count_out, cudaStream_t s) {
  const uint32_t blocks = upper ? (upper + kSpThreads - 1) / kSpThreads : 1;
  k_sparse_count<<<blocks, kSpThreads, 0, s>>>(idx, count, block_counts);
  k_scan_blocks<<<1, 1024, 0, s>>>(block_counts, blocks, count_out);
  k_sparse_fold<<<blocks, kSpThreads, 0, s>>>(idx, val, count, block_counts, make_fixed_mul(r), idx_out, val_out);
  return 3;
}

void launch_scatter(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, Fr* dense,
                    int sm_count, cudaStream_t s) {
  k_scatter<<<blocks_for(upper, 256, sm_count * 8), 256, 0, s>>>(idx, val, count, dense);
}

void launch_check_sorted(const uint32_t* idx, uint32_t n, uint64_t limit, uint32_t* bad, int sm_count, cudaStream_t s) {
  k_check_sorted<<<blocks_for(n, 256, sm_count * 8), 256, 0, s>>>(idx, n, limit, bad);
}

void launch_check_bound(const uint32_t* idx, uint32_t n, uint64_t limit, uint32_t* bad, int sm_count, cudaStream_t s) {
  k_check_bound<<<blocks_for(n, 256, sm_count * 8), 256, 0, s>>>(idx, n, limit, bad);
}

void launch_narrow_idx(const uint64_t* in, uint32_t n, uint32_t* out, uint32_t* bad, int sm_count, cudaStream_t s,
                       uint64_t clamp_below) {
  k_narrow_idx<<<blocks_for(n, 256, sm_count * 8), 256, 0, s>>>(in, n, out, bad, clamp_below);
}

void launch_sd_final(const uint32_t* idx, const Fr* val, const uint32_t* count, const Fr* dense, Fr* out,
                     cudaStream_t s) {
  k_sd_final<<<1, 32, 0, s>>>(idx, val, count, dense, out);
}

}  // namespace zk
