// The two data-movement steps of Einsum::prove ahead of its sumcheck (basicblock/einsum.rs:487-519):
//
//  * permute_evals_by_ranges (einsum.rs:142-198): reorder the variables of an evaluation table, the
//    new order being a list of ranges of old variables;
//  * fix_variables_zkgpt (util/poly.rs:1378-1473): bind the low k variables of a table of signed
//    128-bit integers, out[c] = sum_b eq(r)[b] * t[c 2^k + b].  The reference builds a table of small
//    multiples of eq so that it only adds; here a product of a 32-bit (or 128-bit) integer with a
//    256-bit eq value is 8 (or 32) multiply-adds into a 416-bit accumulator that is reduced once per
//    thread.
#include "internal.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

__device__ __forceinline__ Fr ldg_fr(const Fr* p) {
  const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p)), hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}

struct RangeMap {     // new index bits [dst, dst + len) come from old index bits [src, src + len)
  uint8_t src[40], dst[40], len[40];
  int count;
};

template <class T>
__global__ void __launch_bounds__(256) k_permute_ranges(const T* __restrict__ in, T* __restrict__ out, uint64_t total,
                                                        const __grid_constant__ RangeMap map) {
  for (uint64_t idx_new = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx_new < total;
       idx_new += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t idx_old = 0;
    for (int r = 0; r < map.count; r++)
      idx_old |= ((idx_new >> map.dst[r]) & ((1ull << map.len[r]) - 1)) << map.src[r];
    out[idx_new] = in[idx_old];
  }
}

// acc[i .. 13) += m * e (8 limbs) placed at limb i: two carry chains over the even and the odd limb
// products (each a run of non-overlapping 32x32+64 multiply-adds), then one chain for their carries.
__device__ __forceinline__ void mac_limb(uint32_t (&acc)[13], int i, uint32_t m, const uint32_t* e) {
  const uint32_t c_even = madwide4_c(&acc[i], e[0], e[2], e[4], e[6], m);      // limbs i .. i+7, carry into i+8
  const uint32_t c_odd = madwide4_c(&acc[i + 1], e[1], e[3], e[5], e[7], m);   // limbs i+1 .. i+8, carry into i+9
  uint64_t carry = c_even;
#pragma unroll
  for (int k = i + 8; k < 13; k++) {
    const uint64_t t = (uint64_t)acc[k] + carry + (k == i + 9 ? c_odd : 0u);
    acc[k] = (uint32_t)t;
    carry = t >> 32;
  }
}

// The 416-bit sum of (integer) x (Montgomery-form element) products, reduced: still Montgomery form.
__device__ __forceinline__ Fr reduce_acc(const uint32_t (&acc)[13]) {
  Fr lo, hi = Fr::zero();
#pragma unroll
  for (int i = 0; i < 8; i++) lo.v[i] = acc[i];
#pragma unroll
  for (int i = 0; i < 5; i++) hi.v[i] = acc[8 + i];
  // lo mod p through a Montgomery round trip (inputs below 2^256 are fine); hi * 2^256 = mul(hi, R^2)
  const Fr a = to_mont(from_mont(lo));
  const Fr b = mul(hi, Fr::r2());
  return add(a, b);
}

// Every row enters as t + 2^31, which is a single non-negative 32-bit limb for the quantised values
// this fold is meant for, so the common case needs no sign handling: sum_b eq[b] = 1 turns the
// offset into the constant 2^31 that offset_term() takes off each finished column.  When some lane
// of the warp holds a value outside [-2^31, 2^31) all lanes take the general signed 128-bit path
// for that row (still on t + 2^31).
inline Fr offset_term() {  // host side; passed to the kernels
  Fr x = Fr::zero();
  x.v[0] = 1u << 31;
  return to_mont(x);
}

__device__ __forceinline__ void accumulate_one(uint4 t, bool live, const Fr* __restrict__ eq_b, uint32_t (&acc)[13]) {
  const uint32_t ext = (uint32_t)((int32_t)t.x >> 31);
  const bool small = t.y == ext && t.z == ext && t.w == ext;
  Fr e = Fr::zero();
  if (live) e = ldg_fr(eq_b);
  if (__all_sync(0xffffffffu, small)) {
    mac_limb(acc, 0, t.x ^ 0x80000000u, e.v);
    return;
  }
  // t + 2^31 as a signed 128-bit integer, then its magnitude
  uint64_t s = (uint64_t)t.x + 0x80000000u;
  t.x = (uint32_t)s;
  s = (uint64_t)t.y + (s >> 32);
  t.y = (uint32_t)s;
  s = (uint64_t)t.z + (s >> 32);
  t.z = (uint32_t)s;
  const bool was_neg = (t.w >> 31) != 0;
  t.w += (uint32_t)(s >> 32);
  // a negative value plus 2^31 cannot overflow; a non-negative one gives an unsigned 128-bit magnitude
  const bool neg = was_neg && (t.w >> 31) != 0;
  if (neg) {
    t.x = ~t.x; t.y = ~t.y; t.z = ~t.z; t.w = ~t.w;
    uint64_t c = (uint64_t)t.x + 1;
    t.x = (uint32_t)c;
    c = (uint64_t)t.y + (c >> 32);
    t.y = (uint32_t)c;
    c = (uint64_t)t.z + (c >> 32);
    t.z = (uint32_t)c;
    t.w += (uint32_t)(c >> 32);
    uint32_t m[8];
#pragma unroll
    for (int i = 0; i < 8; i++) m[i] = FrParams::mod(i);
    if (live) (void)sub8(e.v, m, e.v);  // p - eq: the same residue as -eq
  }
  mac_limb(acc, 0, t.x, e.v);
  mac_limb(acc, 1, t.y, e.v);
  mac_limb(acc, 2, t.z, e.v);
  mac_limb(acc, 3, t.w, e.v);
}

// One (column, row range) item: rows [b0, b1) of the column for this lane (first row b0 + first,
// then every step-th); four rows are loaded ahead of the arithmetic.
__device__ __forceinline__ void accumulate_rows(const uint4* __restrict__ t_col, const Fr* __restrict__ eq, uint64_t b0,
                                                uint64_t b1, uint64_t first, uint64_t step, uint32_t (&acc)[13]) {
  for (uint64_t base = b0; base < b1; base += 4 * step) {
    uint4 t[4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const uint64_t b = base + u * step + first;
      live[u] = b < b1;
      t[u] = live[u] ? __ldg(t_col + b) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; u++) accumulate_one(t[u], live[u], eq + base + u * step + first, acc);
  }
}

// Columns of at least 32 rows: one warp per (column, split) item.
__global__ void __launch_bounds__(128) k_int_fold_warp(const uint4* __restrict__ t, const Fr* __restrict__ eq, uint64_t n_rows,
                                                       uint64_t m_cols, uint32_t splits, const Fr offset, Fr* out) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const uint64_t per = n_rows / splits;  // a power of two, at least 32
  for (uint64_t item = warp; item < m_cols * splits; item += warps) {
    const uint64_t c = item % m_cols, s = item / m_cols;
    uint32_t acc[13];
#pragma unroll
    for (int i = 0; i < 13; i++) acc[i] = 0;
    accumulate_rows(t + c * n_rows, eq, s * per, (s + 1) * per, lane, 32, acc);
    const Fr total = warp_sum(reduce_acc(acc));
    if (lane == 0) out[s * m_cols + c] = splits == 1 ? sub(total, offset) : total;
  }
}

// Columns shorter than a warp: one thread per column.
__global__ void __launch_bounds__(128) k_int_fold_thread(const uint4* __restrict__ t, const Fr* __restrict__ eq, uint64_t n_rows,
                                                         uint64_t m_cols, const Fr offset, Fr* out) {
  const uint64_t base = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) & ~31ull;  // the warp's first column
  const int lane = threadIdx.x & 31;
  if (base >= m_cols) return;
  const uint64_t c = base + lane;
  const bool live = c < m_cols;
  uint32_t acc[13];
#pragma unroll
  for (int i = 0; i < 13; i++) acc[i] = 0;
  // every lane walks its own column; lanes past the end walk column 0 and discard the result
  accumulate_rows(t + (live ? c : 0) * n_rows, eq, 0, n_rows, 0, 1, acc);
  const Fr total = sub(reduce_acc(acc), offset);
  if (live) out[c] = total;
}

__global__ void __launch_bounds__(256) k_int_sum_splits(const Fr* __restrict__ partial, uint64_t m_cols, uint32_t splits,
                                                        const Fr offset, Fr* out) {
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= m_cols) return;
  Fr s = partial[c];
  for (uint32_t k = 1; k < splits; k++) s = add(s, partial[(uint64_t)k * m_cols + c]);
  out[c] = sub(s, offset);
}

}  // namespace

// ranges: (start, end) pairs of old variables in their new order; they were validated by the caller.
int launch_permute_ranges(const void* in, void* out, uint32_t n, uint32_t elem_bytes, const uint32_t* ranges,
                          uint32_t n_ranges, int sm_count, cudaStream_t s) {
  RangeMap map;
  map.count = (int)n_ranges;
  uint32_t pos = 0;
  for (uint32_t r = 0; r < n_ranges; r++) {
    map.src[r] = (uint8_t)ranges[2 * r];
    map.len[r] = (uint8_t)(ranges[2 * r + 1] - ranges[2 * r]);
    map.dst[r] = (uint8_t)pos;
    pos += map.len[r];
  }
  const uint64_t total = 1ull << n;
  uint64_t blocks = (total + 255) / 256;
  if (blocks > (uint64_t)sm_count * 16) blocks = (uint64_t)sm_count * 16;
  if (elem_bytes == 32)
    k_permute_ranges<ulonglong4><<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const ulonglong4*>(in),
                                                                   reinterpret_cast<ulonglong4*>(out), total, map);
  else
    k_permute_ranges<uint4><<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out),
                                                              total, map);
  return 1;
}

uint32_t int_fold_splits(uint64_t n_rows, uint64_t m_cols, int sm_count) {
  if (n_rows < 64) return 1;
  uint64_t want = ((uint64_t)sm_count * 16 + m_cols - 1) / m_cols;  // about 16 warps of work per SM
  uint32_t splits = 1;
  while (splits < want && n_rows / (splits * 2) >= 32 && splits < 4096) splits *= 2;
  return splits;
}

// out[c] = sum_b eq[b] * t[c * n_rows + b]; t: signed 128-bit little-endian integers; partial needs
// int_fold_splits() * m_cols elements when that is above 1.  Returns launches.
int launch_int_fold(const void* t, const Fr* eq, uint64_t n_rows, uint64_t m_cols, Fr* partial, Fr* out, int sm_count,
                    cudaStream_t s) {
  const uint4* tt = reinterpret_cast<const uint4*>(t);
  const Fr offset = offset_term();
  if (n_rows < 32) {
    k_int_fold_thread<<<(unsigned)((m_cols + 127) / 128), 128, 0, s>>>(tt, eq, n_rows, m_cols, offset, out);
    return 1;
  }
  const uint32_t splits = int_fold_splits(n_rows, m_cols, sm_count);
  uint64_t blocks = (m_cols * splits + 3) / 4;
  if (blocks > (uint64_t)sm_count * 16) blocks = (uint64_t)sm_count * 16;
  if (splits == 1) {
    k_int_fold_warp<<<(unsigned)blocks, 128, 0, s>>>(tt, eq, n_rows, m_cols, 1, offset, out);
    return 1;
  }
  k_int_fold_warp<<<(unsigned)blocks, 128, 0, s>>>(tt, eq, n_rows, m_cols, splits, offset, partial);
  k_int_sum_splits<<<(unsigned)((m_cols + 255) / 256), 256, 0, s>>>(partial, m_cols, splits, offset, out);
  return 2;
}

}  // namespace zk
