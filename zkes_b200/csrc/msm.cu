// Pippenger multi-scalar multiplication over BN254 G1, for one row or for many rows that share
// the bases (the d_x / d_y loops of kzh2.rs:653-660, kzh3.rs:680-687,743-750).
//
//   1. k_msm_bits     largest magnitude of the sign-folded scalars -> window width W, windows K
//   2. k_msm_digits   signed W-bit digits; MODE 0 counts (row, window, bucket) keys, MODE 1
//                     scatters point indices (sign in bit 31) to their bucket's slots
//   3. k_msm_accumulate  equal chunks of the sorted entry list are summed by one thread each with
//                     mixed additions; a bucket inside one chunk is written directly, pieces of
//                     buckets that cross chunk borders go to per-chunk head / tail slots
//   4. k_msm_fixup    buckets that span chunks: tail of the first chunk + heads of the others
//   5. k_msm_bucket_reduce  sum_j (j+1) B_j per (row, window) by running sums per thread,
//                     a small scalar multiple for the thread's offset, then a block tree
//   6. k_msm_combine  Horner over the windows (W doublings each), Jacobian out
// Small scalars (quantised int8 / int16 weights and activations, negatives stored as r - |v|)
// fold to a few bits, so they use one narrow window: no doublings, few buckets.
#include "msm.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

__device__ __forceinline__ Fr ld_scalar(const Fr* p) {
  const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}

// Canonical value of a Montgomery-form scalar, folded to min(s, r - s); returns the sign.
__device__ __forceinline__ bool fold_scalar(const Fr& mont, uint32_t (&mag)[8]) {
  const Fr c = from_mont(mont);
  uint32_t m[8], d[8];
#pragma unroll
  for (int i = 0; i < 8; i++) m[i] = FrParams::mod(i);
  (void)sub8(d, m, c.v);  // r - s
  // s > r - s  <=>  borrow when computing (r - s) - s
  uint32_t t[8];
  const bool negv = sub8(t, d, c.v) != 0 && !c.is_zero();
#pragma unroll
  for (int i = 0; i < 8; i++) mag[i] = negv ? d[i] : c.v[i];
  return negv;
}

__device__ __forceinline__ int bit_length(const uint32_t (&mag)[8]) {
  int bits = 0;
#pragma unroll
  for (int i = 0; i < 8; i++)
    if (mag[i]) bits = 32 * i + (32 - __clz(mag[i]));
  return bits;
}

// Scalars whose folded magnitude is below 2^30 also have a compact form: a signed 32-bit integer.
// When every scalar of a call has one (quantised weights and activations), the digit passes read
// these 4 bytes instead of converting the 32-byte Montgomery value again.
constexpr int kCompactBits = 30;
constexpr int32_t kNotCompact = INT32_MIN;

// max_out[0]: largest bit length; max_out[1]: largest magnitude among the scalars below 2^32.
__global__ void k_msm_bits(const Fr* __restrict__ scalars, uint64_t total, unsigned int* max_out, int32_t* compact) {
  int best = 0;
  uint32_t best_mag = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t mag[8];
    const bool negv = fold_scalar(ld_scalar(scalars + i), mag);
    const int b = bit_length(mag);
    best = b > best ? b : best;
    if (b <= 32) best_mag = mag[0] > best_mag ? mag[0] : best_mag;
    if (compact) compact[i] = b <= kCompactBits ? (negv ? -(int32_t)mag[0] : (int32_t)mag[0]) : kNotCompact;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const int o = __shfl_down_sync(0xffffffffu, best, off);
    best = o > best ? o : best;
    const uint32_t m = __shfl_down_sync(0xffffffffu, best_mag, off);
    best_mag = m > best_mag ? m : best_mag;
  }
  if ((threadIdx.x & 31) == 0 && best) {
    atomicMax(max_out, (unsigned int)best);
    atomicMax(max_out + 1, best_mag);
  }
}

// Folded magnitude and sign of scalar g, from the compact form when the call has one.
template <bool COMPACT>
__device__ __forceinline__ bool load_mag(const Fr* __restrict__ scalars, const int32_t* __restrict__ compact, uint64_t g,
                                         uint32_t (&mag)[8]) {
  if (COMPACT) {
    const int32_t v = __ldg(compact + g);
#pragma unroll
    for (int i = 1; i < 8; i++) mag[i] = 0;
    mag[0] = v < 0 ? (uint32_t)(-v) : (uint32_t)v;
    return v < 0;
  } else {
    return fold_scalar(ld_scalar(scalars + g), mag);
  }
}

// W-bit field of mag starting at bit `pos` (pos + W may run past 256: zeros).
__device__ __forceinline__ uint32_t bit_field(const uint32_t (&mag)[8], int pos, int w) {
  const int limb = pos >> 5, sh = pos & 31;
  uint64_t v = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    if (i == limb) v |= (uint64_t)mag[i];
    if (i == limb + 1) v |= (uint64_t)mag[i] << 32;
  }
  return (uint32_t)(v >> sh) & ((1u << w) - 1u);
}

template <int MODE, bool COMPACT>  // MODE 0: count keys, 1: scatter entries
__global__ void k_msm_digits(const Fr* __restrict__ scalars, const int32_t* __restrict__ compact,
                             const uint32_t* __restrict__ row_ids, uint64_t n, uint32_t rows,
                             int w, int k_windows, uint32_t* counts_or_cursor, uint32_t* entries) {
  const uint64_t total = row_ids ? n : n * rows;
  const uint32_t half = 1u << (w - 1);
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t mag[8];
    const bool negv = load_mag<COMPACT>(scalars, compact, g, mag);
    // dense rows: scalar g belongs to row g / n; listed rows: the caller names the row of every scalar
    const uint32_t row = row_ids ? row_ids[g] : (uint32_t)(g / n);
    const uint32_t col = row_ids ? (uint32_t)g : (uint32_t)(g - (uint64_t)row * n);
    uint32_t carry = 0;
    for (int k = 0; k < k_windows; k++) {
      uint32_t raw = bit_field(mag, k * w, w) + carry;
      bool dneg = false;
      if (raw > half) {
        raw = (1u << w) - raw;
        dneg = true;
        carry = 1;
      } else {
        carry = 0;
      }
      if (raw == 0) continue;
      const uint32_t key = (row * (uint32_t)k_windows + (uint32_t)k) * half + (raw - 1);
      if (MODE == 0) {
        atomicAdd(counts_or_cursor + key, 1u);
      } else {
        const uint32_t slot = atomicAdd(counts_or_cursor + key, 1u);
        entries[slot] = col | ((negv != dneg) ? 0x80000000u : 0u);
      }
    }
  }
}

// Same two passes for a small key space (at most kSmallKeys buckets in total): keys are counted in
// shared memory first, so the global counters see one atomic per (block, bucket) instead of
// one per digit.  In scatter mode the block reserves a contiguous range per bucket.
constexpr uint32_t kSmallKeys = 4096;

template <int MODE, bool COMPACT>
__global__ void __launch_bounds__(256) k_msm_digits_small(const Fr* __restrict__ scalars, const int32_t* __restrict__ compact,
                                                          const uint32_t* __restrict__ row_ids,
                                                          uint64_t n, uint32_t rows, int w, int k_windows, uint32_t n_keys,
                                                          uint64_t per_block, uint32_t* counts_or_cursor, uint32_t* entries) {
  __shared__ uint32_t hist[kSmallKeys];
  __shared__ uint32_t basepos[kSmallKeys];
  const uint64_t total = row_ids ? n : n * rows;
  const uint32_t half = 1u << (w - 1);
  const uint64_t begin = (uint64_t)blockIdx.x * per_block;
  const uint64_t end = begin + per_block < total ? begin + per_block : total;
  for (uint32_t k = threadIdx.x; k < n_keys; k += blockDim.x) hist[k] = 0;
  __syncthreads();
  for (int pass = 0; pass < (MODE == 0 ? 1 : 2); pass++) {
    for (uint64_t g = begin + threadIdx.x; g < end; g += blockDim.x) {
      uint32_t mag[8];
      const bool negv = load_mag<COMPACT>(scalars, compact, g, mag);
      const uint32_t row = row_ids ? row_ids[g] : (uint32_t)(g / n);
      const uint32_t col = row_ids ? (uint32_t)g : (uint32_t)(g - (uint64_t)row * n);
      uint32_t carry = 0;
      for (int k = 0; k < k_windows; k++) {
        uint32_t raw = bit_field(mag, k * w, w) + carry;
        bool dneg = false;
        if (raw > half) {
          raw = (1u << w) - raw;
          dneg = true;
          carry = 1;
        } else {
          carry = 0;
        }
        if (raw == 0) continue;
        const uint32_t key = (row * (uint32_t)k_windows + (uint32_t)k) * half + (raw - 1);
        if (pass == 0) {
          atomicAdd(hist + key, 1u);
        } else {
          const uint32_t slot = basepos[key] + atomicAdd(hist + key, 1u);
          entries[slot] = col | ((negv != dneg) ? 0x80000000u : 0u);
        }
      }
    }
    __syncthreads();
    if (pass == 0) {
      for (uint32_t k = threadIdx.x; k < n_keys; k += blockDim.x) {
        const uint32_t c = hist[k];
        if (MODE == 0) {
          if (c) atomicAdd(counts_or_cursor + k, c);
        } else {
          basepos[k] = c ? atomicAdd(counts_or_cursor + k, c) : 0;
          hist[k] = 0;
        }
      }
      __syncthreads();
    }
  }
}

__device__ __forceinline__ Affine ld_affine(const Affine* p) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  const uint4 a = __ldg(q), b = __ldg(q + 1), c = __ldg(q + 2), d = __ldg(q + 3);
  Affine r;
  r.x.v[0] = a.x; r.x.v[1] = a.y; r.x.v[2] = a.z; r.x.v[3] = a.w;
  r.x.v[4] = b.x; r.x.v[5] = b.y; r.x.v[6] = b.z; r.x.v[7] = b.w;
  r.y.v[0] = c.x; r.y.v[1] = c.y; r.y.v[2] = c.z; r.y.v[3] = c.w;
  r.y.v[4] = d.x; r.y.v[5] = d.y; r.y.v[6] = d.z; r.y.v[7] = d.w;
  return r;
}

__device__ __forceinline__ void st_xyzz(Xyzz* p, const Xyzz& v) {
  uint4* q = reinterpret_cast<uint4*>(p);
  const Fq* f[4] = {&v.x, &v.y, &v.zz, &v.zzz};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    q[2 * i] = make_uint4(f[i]->v[0], f[i]->v[1], f[i]->v[2], f[i]->v[3]);
    q[2 * i + 1] = make_uint4(f[i]->v[4], f[i]->v[5], f[i]->v[6], f[i]->v[7]);
  }
}
__device__ __forceinline__ Xyzz ld_xyzz(const Xyzz* p) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  Xyzz v;
  Fq* f[4] = {&v.x, &v.y, &v.zz, &v.zzz};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint4 a = q[2 * i], b = q[2 * i + 1];
    f[i]->v[0] = a.x; f[i]->v[1] = a.y; f[i]->v[2] = a.z; f[i]->v[3] = a.w;
    f[i]->v[4] = b.x; f[i]->v[5] = b.y; f[i]->v[6] = b.z; f[i]->v[7] = b.w;
  }
  return v;
}

// First bucket whose range ends after entry e: smallest b with offsets[b + 1] > e.
__device__ __forceinline__ uint32_t bucket_of(const uint32_t* __restrict__ offsets, uint32_t n_buckets, uint32_t e) {
  uint32_t lo = 0, hi = n_buckets - 1;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (offsets[mid + 1] > e) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// The mixed addition with its ten products as calls of one shared routine: the loop body is then a
// few kilobytes instead of forty, which the instruction cache holds (measured 4 % faster on the
// commit of 2^24 points; the inlined form stalled on instruction fetch).
__device__ __noinline__ Fq fq_mul_call(const Fq a, const Fq b) { return mul(a, b); }

__device__ __forceinline__ Xyzz add_mixed_calls(const Xyzz& p, const Affine& q) {
  if (q.is_inf()) return p;
  if (p.is_inf()) return Xyzz::from_affine(q);
  const Fq u2 = fq_mul_call(q.x, p.zz), s2 = fq_mul_call(q.y, p.zzz);
  const Fq pp_ = sub(u2, p.x), r_ = sub(s2, p.y);
  if (pp_.is_zero()) {
    if (!r_.is_zero()) return Xyzz::inf();
    Xyzz d;
    dbl_affine_rare(&d, &q);
    return d;
  }
  Xyzz r;
  const Fq pp = fq_mul_call(pp_, pp_), ppp = fq_mul_call(pp_, pp), q_ = fq_mul_call(p.x, pp);
  r.x = sub(sub(fq_mul_call(r_, r_), ppp), dbl(q_));
  r.y = sub(fq_mul_call(r_, sub(q_, r.x)), fq_mul_call(p.y, ppp));
  r.zz = fq_mul_call(p.zz, pp);
  r.zzz = fq_mul_call(p.zzz, ppp);
  return r;
}

__global__ void __launch_bounds__(128) k_msm_accumulate(const Affine* __restrict__ bases, const uint32_t* __restrict__ gather,
                                                        const uint32_t* __restrict__ entries,
                                                        const uint32_t* __restrict__ offsets, uint32_t n_buckets,
                                                        uint32_t n_entries, uint32_t seg, uint32_t n_chunks,
                                                        Xyzz* bucket_sums, Xyzz* heads, Xyzz* tails) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  const uint32_t begin = c * seg;
  const uint32_t end = (begin + seg < n_entries) ? begin + seg : n_entries;
  uint32_t b = bucket_of(offsets, n_buckets, begin);
  uint32_t b_end = offsets[b + 1];
  bool began_before = offsets[b] < begin;  // the current bucket started in an earlier chunk
  Xyzz acc = Xyzz::inf();
  for (uint32_t e = begin; e < end; e++) {
    if (e == b_end) {  // bucket b is complete
      if (began_before) st_xyzz(heads + c, acc); else st_xyzz(bucket_sums + b, acc);
      acc = Xyzz::inf();
      began_before = false;
      do { b++; b_end = offsets[b + 1]; } while (b_end <= e);
    }
    const uint32_t ent = entries[e];
    const uint32_t col = ent & 0x7fffffffu;
    Affine pt = ld_affine(bases + (gather ? gather[col] : col));
    if (ent & 0x80000000u) pt = neg(pt);
    acc = add_mixed_calls(acc, pt);
  }
  // the bucket in progress at the end of the chunk
  const bool continues = b_end > end;
  if (began_before)
    st_xyzz(heads + c, acc);            // spans the whole chunk, or ends exactly at its end
  else if (continues)
    st_xyzz(tails + c, acc);
  else
    st_xyzz(bucket_sums + b, acc);
}

constexpr uint32_t kFewPieces = 8;
constexpr uint32_t kFixupPartials = 4096;  // partial sums of the grouped fix-up (buckets x groups)

// One thread per bucket: buckets cut into at most kFewPieces pieces are summed in place; longer
// ones are left to the warp-per-bucket kernel below (found through the `many` list).
__global__ void __launch_bounds__(256) k_msm_fixup_few(const uint32_t* __restrict__ offsets, uint32_t n_buckets, uint32_t seg,
                                                       Xyzz* bucket_sums, const Xyzz* heads, const Xyzz* tails,
                                                       uint32_t* many, uint32_t* n_many) {
  const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_buckets) return;
  const uint32_t s = offsets[b], e = offsets[b + 1];
  if (e <= s) return;
  const uint32_t c0 = s / seg, c1 = (e - 1) / seg;
  if (c0 == c1) return;
  if (c1 - c0 >= kFewPieces) {
    many[atomicAdd(n_many, 1u)] = b;
    return;
  }
  Xyzz acc = ld_xyzz(tails + c0);
  for (uint32_t c = c0 + 1; c <= c1; c++) acc = add(acc, ld_xyzz(heads + c));  // one call site: inlined
  st_xyzz(bucket_sums + b, acc);
}

// One warp per listed bucket (those cut into many pieces).
__global__ void __launch_bounds__(128) k_msm_fixup(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ many,
                                                   const uint32_t* __restrict__ n_many, uint32_t seg,
                                                   Xyzz* bucket_sums, const Xyzz* heads, const Xyzz* tails) {
  __shared__ Xyzz sh[4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t total = *n_many;
  for (uint32_t item = blockIdx.x * 4 + warp; item < total; item += gridDim.x * 4) {
  const uint32_t b = many[item];
  const uint32_t s = offsets[b], e = offsets[b + 1];
  const uint32_t c0 = s / seg, c1 = (e - 1) / seg;
  // pieces: tail of chunk c0, heads of chunks c0+1 .. c1
  Xyzz acc = Xyzz::inf();
  for (uint32_t c = c0 + lane; c <= c1; c += 32) {
    const Xyzz h = ld_xyzz(c == c0 ? tails + c : heads + c);
    add_to(&acc, &h);
  }
  sh[warp][lane] = acc;
  __syncwarp();
  for (int off = 16; off > 0; off >>= 1) {
    if (lane < off) {
      add_to(&acc, &sh[warp][lane + off]);
      sh[warp][lane] = acc;
    }
    __syncwarp();
  }
  if (lane == 0) st_xyzz(bucket_sums + b, acc);
  __syncwarp();
  }
}

// Few, long buckets (one narrow window over millions of points): one block per bucket.
__global__ void __launch_bounds__(128) k_msm_fixup_block(const uint32_t* __restrict__ offsets, uint32_t seg,
                                                         Xyzz* bucket_sums, const Xyzz* heads, const Xyzz* tails) {
  __shared__ Xyzz sh[128];
  const uint32_t b = blockIdx.x;
  const uint32_t s = offsets[b], e = offsets[b + 1];
  if (e <= s) return;
  const uint32_t c0 = s / seg, c1 = (e - 1) / seg;
  if (c0 == c1) return;
  Xyzz acc = Xyzz::inf();
  for (uint32_t c = c0 + threadIdx.x; c <= c1; c += blockDim.x) {
    const Xyzz h = ld_xyzz(c == c0 ? tails + c : heads + c);
    add_to(&acc, &h);
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (uint32_t off = blockDim.x >> 1; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      add_to(&acc, &sh[threadIdx.x + off]);
      sh[threadIdx.x] = acc;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) st_xyzz(bucket_sums + b, acc);
}

// Very long buckets (a narrow window over millions of points, or the single bucket of an all-ones MSM): the
// pieces of a bucket are shared by `groups` blocks, each leaving a partial sum, and a second small launch adds
// the partial sums of every bucket.
__global__ void __launch_bounds__(128) k_msm_fixup_groups(const uint32_t* __restrict__ offsets, uint32_t seg, uint32_t groups,
                                                          const Xyzz* heads, const Xyzz* tails, Xyzz* partial) {
  __shared__ Xyzz sh[128];
  const uint32_t b = blockIdx.x, g = blockIdx.y;
  const uint32_t s = offsets[b], e = offsets[b + 1];
  Xyzz acc = Xyzz::inf();
  if (e > s) {
    const uint32_t c0 = s / seg, c1 = (e - 1) / seg;
    if (c0 != c1)
      for (uint32_t c = c0 + g + groups * threadIdx.x; c <= c1; c += groups * blockDim.x) {
        const Xyzz h = ld_xyzz(c == c0 ? tails + c : heads + c);
        add_to(&acc, &h);
      }
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (uint32_t off = blockDim.x >> 1; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      add_to(&acc, &sh[threadIdx.x + off]);
      sh[threadIdx.x] = acc;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) st_xyzz(partial + (size_t)b * groups + g, acc);
}

__global__ void __launch_bounds__(32) k_msm_fixup_groups_final(const uint32_t* __restrict__ offsets, uint32_t seg, uint32_t groups,
                                                               const Xyzz* partial, Xyzz* bucket_sums) {
  __shared__ Xyzz sh[32];
  const uint32_t b = blockIdx.x;
  const uint32_t s = offsets[b], e = offsets[b + 1];
  if (e <= s || s / seg == (e - 1) / seg) return;  // the accumulation wrote this bucket directly
  Xyzz acc = Xyzz::inf();
  for (uint32_t g = threadIdx.x; g < groups; g += 32) {
    const Xyzz h = ld_xyzz(partial + (size_t)b * groups + g);
    add_to(&acc, &h);
  }
  sh[threadIdx.x] = acc;
  __syncwarp();
  for (int off = 16; off > 0; off >>= 1) {
    if (threadIdx.x < (unsigned)off) {
      add_to(&acc, &sh[threadIdx.x + off]);
      sh[threadIdx.x] = acc;
    }
    __syncwarp();
  }
  if (threadIdx.x == 0) st_xyzz(bucket_sums + b, acc);
}

// One block per (row, window): sum_j (j + 1) * B_j over `half` buckets.
__global__ void __launch_bounds__(256) k_msm_bucket_reduce(const Xyzz* __restrict__ bucket_sums, uint32_t half,
                                                           Xyzz* window_sums) {
  extern __shared__ unsigned char sh_raw[];
  Xyzz* sh = reinterpret_cast<Xyzz*>(sh_raw);
  const Xyzz* B = bucket_sums + (size_t)blockIdx.x * half;
  const uint32_t per = (half + blockDim.x - 1) / blockDim.x;
  const uint32_t lo = threadIdx.x * per;
  const uint32_t hi = (lo + per < half) ? lo + per : half;
  Xyzz running = Xyzz::inf(), acc = Xyzz::inf();
  if (lo < half) {
    for (uint32_t j = hi; j-- > lo;) {
      const Xyzz bj = ld_xyzz(B + j);
      add_to(&running, &bj);
      add_to(&acc, &running);
    }
    if (lo) {
      const Xyzz m = mul_small(running, lo);
      add_to(&acc, &m);
    }
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (uint32_t off = blockDim.x >> 1; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      add_to(&acc, &sh[threadIdx.x + off]);
      sh[threadIdx.x] = acc;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) st_xyzz(window_sums + blockIdx.x, acc);
}

// Many short rows (the d_x / d_y rows of a commitment: thousands of (row, window) items of at most
// 256 buckets): a block per item leaves most of its additions to idle lanes.  Here eight lanes share
// an item and four items a warp.  Lane l takes `per` consecutive buckets: running sums give its local
// weighted sum A_l = sum_j (j - lo + 1) B_j and its plain sum R_l.  The item's result is
// sum_l A_l + per * sum_{l >= 1} S_l with S_l = sum_{u >= l} R_u (a suffix scan over the eight lanes), so
// every lane doubles its own S_l log2(per) times, adds A_l, and one three-level tree finishes.
constexpr int kRowLanes = 8;
__global__ void __launch_bounds__(128) k_msm_bucket_reduce_rows(const Xyzz* __restrict__ bucket_sums, uint32_t half,
                                                               uint32_t n_items, Xyzz* window_sums) {
  __shared__ Xyzz sh[128];
  const uint32_t t = threadIdx.x, l = t & (kRowLanes - 1);
  const uint32_t item = blockIdx.x * (128 / kRowLanes) + t / kRowLanes;
  const bool live = item < n_items;
  const uint32_t per = half / kRowLanes;  // a power of two, at least 1
  const Xyzz* B = bucket_sums + (size_t)(live ? item : 0) * half;
  Xyzz running = Xyzz::inf(), acc = Xyzz::inf();
  if (live) {
    const uint32_t lo = l * per;
    for (uint32_t j = lo + per; j-- > lo;) {
      const Xyzz bj = ld_xyzz(B + j);
      add_to(&running, &bj);
      add_to(&acc, &running);
    }
  }
  // inclusive suffix scan of the running sums over the item's lanes
  sh[t] = running;
  __syncwarp();
#pragma unroll
  for (uint32_t off = 1; off < kRowLanes; off <<= 1) {
    Xyzz other = Xyzz::inf();
    if (l + off < kRowLanes) other = sh[t + off];
    __syncwarp();
    add_to(&running, &other);
    sh[t] = running;
    __syncwarp();
  }
  // lane l >= 1 contributes per * S_l
  if (l == 0) running = Xyzz::inf();
  for (uint32_t k = per; k > 1; k >>= 1) dbl_in_place(&running);
  add_to(&acc, &running);
  sh[t] = acc;
  __syncwarp();
#pragma unroll
  for (uint32_t off = kRowLanes / 2; off > 0; off >>= 1) {
    Xyzz other = Xyzz::inf();
    if (l < off) other = sh[t + off];
    __syncwarp();
    add_to(&acc, &other);
    sh[t] = acc;
    __syncwarp();
  }
  if (live && l == 0) st_xyzz(window_sums + item, acc);
}

__global__ void k_msm_combine(const Xyzz* __restrict__ window_sums, uint32_t rows, int w, int k_windows, Jacobian* out) {
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  Xyzz acc = Xyzz::inf();
  for (int k = k_windows - 1; k >= 0; k--) {
    for (int i = 0; i < w; i++) dbl_in_place(&acc);
    const Xyzz ws = ld_xyzz(window_sums + (size_t)row * k_windows + k);
    add_to(&acc, &ws);
  }
  out[row] = to_jacobian(acc);
}

// 64-bit total of the per-bucket counts (the 32-bit prefix sums would wrap silently past 2^32).
__global__ void k_total64(const uint32_t* __restrict__ counts, uint32_t n, unsigned long long* total) {
  unsigned long long s = 0;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) s += counts[i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
  if ((threadIdx.x & 31) == 0 && s) atomicAdd(total, s);
}

__global__ void k_set_infinity(Jacobian* out, uint32_t rows) {
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < rows) out[row] = to_jacobian(Xyzz::inf());
}

// ---- Sums of selected SRS points: the commitment of a selection polynomial (every listed entry is one).
// sparse_kzh2_commit / sparse_kzh3_commit (sparse_kzh2.rs:27-80, sparse_kzh3.rs:45-110) with all values one are
// C = sum_i h_full[idx_i] and d_x[r] = sum_{i in row r} h_mid[idx_i mod 2^low_bits], row r = idx >> low_bits.  With the
// indices in non-decreasing order a row is a contiguous run of the list, so the digit, sort and bucket passes of
// the general MSM are not needed: sixteen lanes take a row, each lane sums its share with mixed additions, a tree over
// the lanes (through shared memory) finishes the row, and the same walk adds the row's share of C.
constexpr int kSelLanes = 16;  // lanes per row (a full warp per row measured 20-35 % slower: twice the tree additions)

__device__ __forceinline__ uint32_t sel_lower_bound(const uint32_t* __restrict__ idx, uint32_t n, uint64_t key) {
  uint32_t lo = 0, hi = n;  // first position with idx >= key
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (idx[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(128) k_select_sums(const Affine* __restrict__ full, const Affine* __restrict__ mid,
                                                     const uint32_t* __restrict__ idx, uint32_t n, uint32_t low_bits,
                                                     uint32_t rows, Jacobian* d_x, Xyzz* c_partial) {
  const uint32_t group = (blockIdx.x * blockDim.x + threadIdx.x) / kSelLanes, gl = threadIdx.x % kSelLanes;
  uint32_t lo = 0, hi = 0;
  if (group < rows) {
    lo = sel_lower_bound(idx, n, (uint64_t)group << low_bits);
    hi = sel_lower_bound(idx, n, ((uint64_t)group + 1) << low_bits);
  }
  const uint32_t mask = low_bits >= 32 ? 0xffffffffu : (1u << low_bits) - 1u;
  Xyzz acc_c = Xyzz::inf(), acc_r = Xyzz::inf();
  for (uint32_t i = lo + gl; i < hi; i += kSelLanes) {
    const uint32_t v = idx[i];
    acc_c = add_mixed_calls(acc_c, ld_affine(full + v));
    acc_r = add_mixed_calls(acc_r, ld_affine(mid + (v & mask)));
  }
  // The lanes' shares of a row: a tree through shared memory.  The time of this kernel follows the number of
  // warp-wide additions it issues, so the additions of a level are packed into as few warps as they fill: the row
  // sums' pairs take the first threads of the block, C's pairs the next, and whole warps sit a level out
  // (128, 64, 32 and 16 additions for the four levels, against two additions by every warp at every level).
  __shared__ Xyzz sh[2 * 128];  // [0, 128): shares of the rows' sums; [128, 256): shares of C
  sh[threadIdx.x] = acc_r;
  sh[128 + threadIdx.x] = acc_c;
  __syncthreads();
  constexpr int kRowsPerBlock = 128 / kSelLanes;
#pragma unroll 1
  for (int off = kSelLanes / 2; off > 0; off >>= 1) {
    const int per_kind = kRowsPerBlock * off;  // additions of this level for one of the two sums
    if ((int)threadIdx.x < 2 * per_kind) {
      const int kind = (int)threadIdx.x / per_kind, t = (int)threadIdx.x % per_kind;
      Xyzz* at = sh + kind * 128 + (t / off) * kSelLanes + (t % off);
      add_to(at, at + off);
    }
    __syncthreads();
  }
  acc_r = sh[threadIdx.x];
  Xyzz* sh_c = sh + 128;
  if (group < rows && gl == 0) d_x[group] = to_jacobian(acc_r);
  // the shares of C of the block's rows: one more tree, by the first lanes of the block
  constexpr unsigned kRowMask = (1u << kRowsPerBlock) - 1u;
  __syncthreads();  // sh_c[kSelLanes k] holds row k's share
  if (threadIdx.x < kRowsPerBlock) {
    Xyzz v = sh_c[kSelLanes * threadIdx.x];
    __syncwarp(kRowMask);
#pragma unroll 1
    for (int off = kRowsPerBlock / 2; off > 0; off >>= 1) {
      sh_c[threadIdx.x] = v;
      __syncwarp(kRowMask);
      if ((int)threadIdx.x < off) add_to(&v, &sh_c[threadIdx.x + off]);
      __syncwarp(kRowMask);
    }
    if (threadIdx.x == 0) st_xyzz(c_partial + blockIdx.x, v);
  }
}

// C = the sum of the blocks' shares (one block).
__global__ void __launch_bounds__(256) k_select_total(const Xyzz* __restrict__ c_partial, uint32_t rows, Jacobian* c_out) {
  __shared__ Xyzz sh[256];
  Xyzz acc = Xyzz::inf();
  for (uint32_t r = threadIdx.x; r < rows; r += blockDim.x) {
    const Xyzz v = ld_xyzz(c_partial + r);
    add_to(&acc, &v);
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
#pragma unroll 1
  for (int off = 128; off > 0; off >>= 1) {
    if ((int)threadIdx.x < off) {
      const Xyzz v = sh[threadIdx.x + off];
      add_to(&acc, &v);
      sh[threadIdx.x] = acc;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *c_out = to_jacobian(acc);
}

}  // namespace

// Window width for n points per row whose scalars have at most max_bits magnitude bits.
static int pick_window(uint64_t n, uint32_t rows, int max_bits) {
  int lg = 0;
  while ((1ull << (lg + 1)) <= n) lg++;
  // a row costs windows * (n + 2 * 2^(w-1)) additions; with many rows the buckets (128 bytes each, per
  // row and window) also have to fit in memory, so rows use a narrower window
  int w = rows > 1 ? lg - 4 : lg - 2;
  if (w > 16) w = 16;
  if (w < 3) w = 3;
  if (w > max_bits + 1) w = max_bits + 1;
  if (w < 2) w = 2;
  return w;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

int msm_run(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const Fr* scalars, uint64_t n, uint32_t rows,
            Jacobian* out_dev, MsmStats* stats, MsmPrep* prep) {
  return msm_run_rows(ctx, bases, gather, nullptr, scalars, n, rows, out_dev, stats, prep);
}

// Signed-digit windows needed for magnitudes up to max_mag: k digits in (-half, half] reach
// half * (1 + 2^w + ... + 2^(w (k - 1))).
static int windows_for(uint32_t max_mag, int w) {
  const uint64_t half = 1ull << (w - 1);
  uint64_t reach = 0;
  int k = 0;
  do {
    reach = (reach << w) + half;
    k++;
  } while (reach < max_mag);
  return k;
}

// row_ids == nullptr: `rows` dense rows of n scalars each over the same n bases.  Otherwise: n scalars in
// all, scalar i contributes scalars[i] * bases[gather ? gather[i] : i] to output row row_ids[i] < rows.
int msm_run_rows(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const uint32_t* row_ids, const Fr* scalars,
                 uint64_t n, uint32_t rows, Jacobian* out_dev, MsmStats* stats, MsmPrep* prep) {
  cudaStream_t s = ctx->stream;
  const uint64_t total = row_ids ? n : n * rows;
  const int sm = ctx->sm_count;
  if (rows == 0) return 0;
  if (n == 0) {
    k_set_infinity<<<(rows + 127) / 128, 128, 0, s>>>(out_dev, rows);
    ctx->launches++;
    return 0;
  }
  if (n >= (1ull << 31)) return fail(-1, "msm: at most 2^31 - 1 points per row");
  // ---- pass 1: scalar magnitude (and the compact form of small scalars); a caller that runs several
  // MSMs over the same scalars passes `prep` and the pass runs once
  unsigned int max_bits = 0;
  uint32_t max_mag = 0;
  const int32_t* compact = nullptr;
  if (prep && prep->valid && prep->scalars == scalars && prep->total == total) {
    max_bits = prep->max_bits;
    max_mag = prep->max_mag;
    compact = prep->compact;
  } else {
    unsigned int* d_bits = ctx->rs.sink.counter + 8;  // spare words of the context's counter block
    int32_t* cbuf = nullptr;
    int crc = ctx->reserve_cmp(total * 4 + 256, (void**)&cbuf);
    if (crc) return crc;
    ZK_CUDA(cudaMemsetAsync(d_bits, 0, 8, s));
    k_msm_bits<<<sm * 8, 256, 0, s>>>(scalars, total, d_bits, cbuf);
    ctx->launches++;
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, d_bits, 8, cudaMemcpyDeviceToHost, s));
    ZK_CUDA(cudaStreamSynchronize(s));
    unsigned int two[2];
    memcpy(two, ctx->host_small, 8);
    max_bits = two[0];
    max_mag = two[1];
    if (max_bits <= (unsigned)kCompactBits) compact = cbuf;
    if (prep) {
      prep->valid = true;
      prep->scalars = scalars;
      prep->total = total;
      prep->max_bits = max_bits;
      prep->max_mag = max_mag;
      prep->compact = compact;
    }
  }
  if (max_bits == 0) {
    k_set_infinity<<<(rows + 127) / 128, 128, 0, s>>>(out_dev, rows);
    ctx->launches++;
    return 0;
  }
  const int w = pick_window(row_ids ? (n / rows ? n / rows : 1) : n, rows, (int)max_bits);
  // small scalars: the exact largest magnitude is known, which can save the window that would only
  // hold carries (int8 values reach 128 = one 8-bit signed digit)
  const int k_windows = compact ? windows_for(max_mag, w) : ((int)max_bits + 1 + w - 1) / w;
  const uint32_t half = 1u << (w - 1);
  const uint64_t n_buckets64 = (uint64_t)rows * k_windows * half;
  if (n_buckets64 >= (1ull << 31)) return fail(-1, "msm: %llu buckets exceed the 32-bit key space; split the rows", (unsigned long long)n_buckets64);
  const uint32_t n_buckets = (uint32_t)n_buckets64;

  // ---- scratch layout (second scratch region of the context; the first holds caller data)
  // worst case: every scalar has a non-zero digit in every window; small scalars have fewer, and the
  // real total is checked after the count pass (entry slots are 32-bit)
  uint64_t max_entries = total * (uint64_t)k_windows;
  if (max_entries > 0xffffffffull) max_entries = 0xffffffffull;
  size_t need = align256((n_buckets + 2) * 4ull) * 2 + align256(scan_scratch_elems(n_buckets + 1) * 4) +
                align256((size_t)n_buckets * sizeof(Xyzz)) + align256((size_t)rows * k_windows * sizeof(Xyzz)) + 4096;
  char* base = nullptr;
  // entries and chunk slots are sized after the count pass; reserve the worst case now
  uint64_t chunk_guess = max_entries / 32 + 1;
  if (chunk_guess > (1u << 20)) chunk_guess = 1u << 20;
  need += align256(max_entries * 4) + 2 * align256((chunk_guess + 1) * sizeof(Xyzz)) + align256((size_t)kFixupPartials * sizeof(Xyzz));
  int rc = ctx->reserve_aux(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += align256(bytes); return p; };
  uint32_t* offsets = (uint32_t*)take((n_buckets + 2) * 4ull);
  uint32_t* cursor = (uint32_t*)take((n_buckets + 2) * 4ull);
  uint32_t* scan_tmp = (uint32_t*)take(scan_scratch_elems(n_buckets + 1) * 4);
  Xyzz* bucket_sums = (Xyzz*)take((size_t)n_buckets * sizeof(Xyzz));
  Xyzz* window_sums = (Xyzz*)take((size_t)rows * k_windows * sizeof(Xyzz));
  uint32_t* entries = (uint32_t*)take(max_entries * 4);
  Xyzz* heads = (Xyzz*)take((chunk_guess + 1) * sizeof(Xyzz));
  Xyzz* tails = (Xyzz*)take((chunk_guess + 1) * sizeof(Xyzz));
  Xyzz* fix_part = (Xyzz*)take((size_t)kFixupPartials * sizeof(Xyzz));

  // ---- pass 2: count, scan, scatter
  ZK_CUDA(cudaMemsetAsync(offsets, 0, (n_buckets + 2) * 4ull, s));
  const bool small_keys = n_buckets <= kSmallKeys;
  uint32_t dig_blocks = (uint32_t)((total + 4095) / 4096);
  if (dig_blocks > (uint32_t)sm * 8) dig_blocks = sm * 8;
  const uint64_t per_block = (total + dig_blocks - 1) / dig_blocks;
  if (small_keys) {
    if (compact)
      k_msm_digits_small<0, true><<<dig_blocks, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, n_buckets, per_block, offsets, nullptr);
    else
      k_msm_digits_small<0, false><<<dig_blocks, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, n_buckets, per_block, offsets, nullptr);
  } else {
    if (compact)
      k_msm_digits<0, true><<<sm * 8, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, offsets, nullptr);
    else
      k_msm_digits<0, false><<<sm * 8, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, offsets, nullptr);
  }
  ctx->launches++;
  unsigned long long* d_total = reinterpret_cast<unsigned long long*>(ctx->rs.sink.counter + 10);
  ZK_CUDA(cudaMemsetAsync(d_total, 0, 8, s));
  k_total64<<<sm * 4, 256, 0, s>>>(offsets, n_buckets, d_total);
  ctx->launches++;
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, d_total, 8, cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  unsigned long long total64 = 0;
  memcpy(&total64, ctx->host_small, 8);
  if (total64 > 0xffffffffull) return fail(-1, "msm: %llu digit entries exceed 2^32 - 1; split the call", total64);
  ctx->launches += exclusive_scan_u32(offsets, n_buckets, scan_tmp, true, s);
  ZK_CUDA(cudaMemcpyAsync(cursor, offsets, (n_buckets + 1) * 4ull, cudaMemcpyDeviceToDevice, s));
  if (small_keys) {
    if (compact)
      k_msm_digits_small<1, true><<<dig_blocks, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, n_buckets, per_block, cursor, entries);
    else
      k_msm_digits_small<1, false><<<dig_blocks, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, n_buckets, per_block, cursor, entries);
  } else {
    if (compact)
      k_msm_digits<1, true><<<sm * 8, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, cursor, entries);
    else
      k_msm_digits<1, false><<<sm * 8, 256, 0, s>>>(scalars, compact, row_ids, n, rows, w, k_windows, cursor, entries);
  }
  ctx->launches++;
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, offsets + n_buckets, 4, cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  uint32_t n_entries = 0;
  memcpy(&n_entries, ctx->host_small, 4);

  // ---- accumulate
  ZK_CUDA(cudaMemsetAsync(bucket_sums, 0, (size_t)n_buckets * sizeof(Xyzz), s));
  if (n_entries) {
    uint32_t n_chunks = n_entries / 32 + 1;
    if (n_chunks > chunk_guess) n_chunks = (uint32_t)chunk_guess;
    const uint32_t seg = (n_entries + n_chunks - 1) / n_chunks;
    n_chunks = (n_entries + seg - 1) / seg;
    k_msm_accumulate<<<(n_chunks + 127) / 128, 128, 0, s>>>(bases, gather, entries, offsets, n_buckets, n_entries, seg,
                                                           n_chunks, bucket_sums, heads, tails);
    // pieces per bucket on average; from a few hundred on, one block per bucket is a long serial chain
    const uint32_t avg_pieces = n_chunks / n_buckets;
    uint32_t groups = (avg_pieces + 255) / 256;
    if (n_buckets <= kFixupPartials && groups > kFixupPartials / n_buckets) groups = kFixupPartials / n_buckets;
    if (n_buckets <= 8192 && n_buckets <= kFixupPartials && groups >= 2) {
      k_msm_fixup_groups<<<dim3(n_buckets, groups), 128, 0, s>>>(offsets, seg, groups, heads, tails, fix_part);
      k_msm_fixup_groups_final<<<n_buckets, 32, 0, s>>>(offsets, seg, groups, fix_part, bucket_sums);
      ctx->launches++;
    } else if (n_buckets <= 8192) {
      k_msm_fixup_block<<<n_buckets, 128, 0, s>>>(offsets, seg, bucket_sums, heads, tails);
    } else {
      // cursor[] is free again after the scatter: reuse it as the list of long buckets
      uint32_t* n_many = ctx->rs.sink.counter + 12;
      ZK_CUDA(cudaMemsetAsync(n_many, 0, 4, s));
      k_msm_fixup_few<<<(n_buckets + 255) / 256, 256, 0, s>>>(offsets, n_buckets, seg, bucket_sums, heads, tails, cursor, n_many);
      k_msm_fixup<<<sm * 4, 128, 0, s>>>(offsets, cursor, n_many, seg, bucket_sums, heads, tails);
      ctx->launches++;
    }
    ctx->launches += 2;
  }
  // ---- reduce buckets, combine windows
  // buckets per thread: the running sums cost 2 additions per bucket, the thread's offset multiple and
  // the block tree are per-thread overhead, so threads take up to 32 buckets while enough threads remain
  uint32_t per_thread = 4;
  while (per_thread < 32 && (uint64_t)rows * k_windows * (half / (per_thread * 2)) >= 100000) per_thread *= 2;
  uint32_t threads = half / per_thread;
  if (threads < 32) threads = 32;
  if (threads > 256) threads = 256;
  const uint32_t n_items = rows * (uint32_t)k_windows;
  if (n_items >= 1024 && half >= kRowLanes && half <= 256)
    k_msm_bucket_reduce_rows<<<(n_items + 15) / 16, 128, 0, s>>>(bucket_sums, half, n_items, window_sums);
  else
    k_msm_bucket_reduce<<<n_items, threads, threads * sizeof(Xyzz), s>>>(bucket_sums, half, window_sums);
  k_msm_combine<<<(rows + 63) / 64, 64, 0, s>>>(window_sums, rows, w, k_windows, out_dev);
  ctx->launches += 2;
  ZK_CUDA(cudaGetLastError());
  ctx->msm_entries_sum += n_entries;
  ctx->msm_bucket_sum += n_buckets;
  ctx->msm_calls++;
  if (stats) {
    stats->window_bits = w;
    stats->windows = k_windows;
    stats->entries = n_entries;
    stats->buckets = n_buckets;
    stats->max_bits = (int)max_bits;
  }
  return 0;
}

// C (out_dev[rows]) and d_x (out_dev[0 .. rows)) of a selection polynomial over n indices in non-decreasing order
// (device, 32-bit), below rows << low_bits.  scratch: rows Xyzz elements of device memory.
int msm_select_sums(zk_ctx* ctx, const Affine* full, const Affine* mid, const uint32_t* idx_dev, uint32_t n, uint32_t low_bits,
                    uint32_t rows, Jacobian* out_dev, void* scratch) {
  cudaStream_t s = ctx->stream;
  Xyzz* partial = reinterpret_cast<Xyzz*>(scratch);
  const uint32_t threads = rows * kSelLanes;
  const uint32_t blocks = (threads + 127) / 128;
  k_select_sums<<<blocks, 128, 0, s>>>(full, mid, idx_dev, n, low_bits, rows, out_dev, partial);
  k_select_total<<<1, 256, 0, s>>>(partial, blocks, out_dev + rows);
  ctx->launches += 2;
  ctx->msm_calls += 2;
  ctx->msm_entries_sum += 2ull * n;
  ctx->msm_bucket_sum += rows + 1;
  ZK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace zk
