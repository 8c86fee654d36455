// Fixed-base generation of structured reference strings: out[i] = (alpha * prod_f tau_f[digits_f(i)]) * g,
// the h_xy / h_y / h_xyz / h_yz / h_z vectors of setup_kzh2_srs (kzh2.rs:502-555) and setup_kzh3_srs
// (kzh3.rs:463-563).  A table of d * 2^(16 w) * g (w < 16, 1 <= d <= 2^15) turns every scalar
// multiplication into at most 16 mixed additions of table entries selected by signed 16-bit digits.
#include "msm.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

constexpr int kFbWindows = 16;
constexpr uint32_t kFbHalf = 1u << 15;

__global__ void k_fb_powers(const Affine g, Affine* powers) {
  if (threadIdx.x || blockIdx.x) return;
  Xyzz p = Xyzz::from_affine(g);
  for (int w = 0; w < kFbWindows; w++) {
    powers[w] = to_affine(p);
    for (int i = 0; i < 16; i++) p = dbl(p);
  }
}

__global__ void __launch_bounds__(128) k_fb_table(const Affine* __restrict__ powers, Affine* table) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= kFbWindows * kFbHalf) return;
  const uint32_t w = t / kFbHalf, d = t % kFbHalf + 1;
  table[t] = to_affine(mul_small(Xyzz::from_affine(powers[w]), d));
}

struct FbFactors {
  const Fr* table[3];
  uint32_t shift[3];
  uint32_t mask[3];
  int count;
  int has_alpha;
  Fr alpha;
};

__global__ void __launch_bounds__(128) k_fb_generate(const Affine* __restrict__ table, const FbFactors f, uint64_t start,
                                                     uint64_t count, Affine* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t g = start + i;  // index into the whole vector; out holds the slab [start, start + count)
    Fr s = f.has_alpha ? f.alpha : Fr::one();
    for (int k = 0; k < f.count; k++) s = mul(s, f.table[k][(g >> f.shift[k]) & f.mask[k]]);
    const Fr c = from_mont(s);
    uint32_t m[8], d[8], t[8], mag[8];
#pragma unroll
    for (int k = 0; k < 8; k++) m[k] = FrParams::mod(k);
    (void)sub8(d, m, c.v);
    const bool negv = sub8(t, d, c.v) != 0;
#pragma unroll
    for (int k = 0; k < 8; k++) mag[k] = negv ? d[k] : c.v[k];
    Xyzz acc = Xyzz::inf();
    uint32_t carry = 0;
#pragma unroll 1
    for (int w = 0; w < kFbWindows; w++) {
      uint32_t raw = ((mag[w >> 1] >> ((w & 1) * 16)) & 0xffffu) + carry;
      bool dneg = false;
      if (raw > kFbHalf) {
        raw = 0x10000u - raw;
        dneg = true;
        carry = 1;
      } else {
        carry = 0;
      }
      if (raw == 0) continue;
      Affine pt = table[(uint32_t)w * kFbHalf + raw - 1];
      if (negv != dneg) pt = neg(pt);
      acc = add_mixed(acc, pt);
    }
    out[i] = to_affine(acc);
  }
}

}  // namespace

size_t fixed_base_table_bytes() { return (size_t)(kFbWindows * kFbHalf + kFbWindows) * sizeof(Affine); }

// table_mem: fixed_base_table_bytes() of device scratch.  Returns launches.
int fixed_base_build_table(const Affine& g, void* table_mem, cudaStream_t s) {
  Affine* powers = reinterpret_cast<Affine*>(table_mem);
  Affine* table = powers + kFbWindows;
  k_fb_powers<<<1, 32, 0, s>>>(g, powers);
  k_fb_table<<<(kFbWindows * kFbHalf + 127) / 128, 128, 0, s>>>(powers, table);
  return 2;
}

// out[i] = (alpha * prod_k tables[k][((start + i) >> shift_k) & (2^bits_k - 1)]) * g for i < count; shift_k is
// the sum of the earlier factors' bits (factor 0 indexes the lowest bits).  Device pointers.
int fixed_base_generate(const void* table_mem, int n_factors, const Fr* const* tables, const uint32_t* bits,
                        const Fr* alpha, uint64_t start, uint64_t count, Affine* out, int sm_count, cudaStream_t s) {
  FbFactors f;
  uint32_t shift = 0;
  for (int k = 0; k < 3; k++) {
    f.table[k] = k < n_factors ? tables[k] : nullptr;
    f.shift[k] = shift;
    f.mask[k] = k < n_factors ? (uint32_t)((1ull << bits[k]) - 1) : 0;
    if (k < n_factors) shift += bits[k];
  }
  f.count = n_factors;
  f.has_alpha = alpha ? 1 : 0;
  f.alpha = alpha ? *alpha : Fr::one();
  uint64_t blocks = (count + 127) / 128;
  if (blocks > (uint64_t)sm_count * 16) blocks = sm_count * 16;
  k_fb_generate<<<(unsigned)blocks, 128, 0, s>>>(reinterpret_cast<const Affine*>(table_mem) + kFbWindows, f, start, count, out);
  return 1;
}

}  // namespace zk
