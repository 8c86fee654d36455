// arkworks' compressed encoding of G1 points (ark-serialize, short Weierstrass): 32 bytes, x as a
// little-endian integer, bit 7 of the last byte set when y is the larger of {y, q - y}, bit 6 set for
// the point at infinity.  It is what the reference absorbs into the transcript for a KZH3
// commitment (kzh3.rs:406-411, util/serialization.rs:14-21) and what its SRS files hold
// (crypto/srs_storage.rs:15-58).  Decompression takes a square root per point
// (q = 3 mod 4: y = (x^3 + 3)^((q+1)/4)), which is why it is worth a kernel for SRS-sized vectors.
#include "../../include/zkb200.h"
#include "ctx.hpp"
#include "ec.cuh"

using namespace zk;

namespace {

struct Limbs8 {
  uint32_t v[8];
};

// a > b on canonical 256-bit integers
__device__ __forceinline__ bool gt256(const uint32_t* a, const uint32_t* b) {
  uint32_t d[8];
  return sub8(d, b, a) != 0;  // b - a borrows exactly when a > b
}

__global__ void __launch_bounds__(128) k_g1_compress(const Affine* __restrict__ in, uint64_t n, uint4* __restrict__ out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const Affine p = in[i];
    uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (p.is_inf()) {
      w[7] = 0x40000000u;
    } else {
      const Fq x = from_mont(p.x), y = from_mont(p.y);
      uint32_t m[8], neg_y[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {
        m[k] = FqParams::mod(k);
        w[k] = x.v[k];
      }
      (void)sub8(neg_y, m, y.v);
      if (gt256(y.v, neg_y)) w[7] |= 0x80000000u;
    }
    out[2 * i] = make_uint4(w[0], w[1], w[2], w[3]);
    out[2 * i + 1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// bad: set to 1 + (index of some invalid encoding) when one is met
__global__ void __launch_bounds__(128) k_g1_decompress(const uint4* __restrict__ in, uint64_t n, const Limbs8 exponent,
                                                       Affine* __restrict__ out, unsigned long long* bad) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint4 lo = in[2 * i], hi = in[2 * i + 1];
    uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    const bool flag_neg = (w[7] >> 31) != 0, flag_inf = ((w[7] >> 30) & 1u) != 0;
    w[7] &= 0x3fffffffu;
    Affine p;
    p.x = Fq::zero();
    p.y = Fq::zero();
    uint32_t m[8], d[8];
#pragma unroll
    for (int k = 0; k < 8; k++) m[k] = FqParams::mod(k);
    bool ok = true;
    if (flag_inf) {
      ok = !flag_neg && (w[0] | w[1] | w[2] | w[3] | w[4] | w[5] | w[6] | w[7]) == 0;
    } else if (sub8(d, w, m) == 0) {
      ok = false;  // x >= q
    } else {
      Fq xr;
#pragma unroll
      for (int k = 0; k < 8; k++) xr.v[k] = w[k];
      const Fq x = to_mont(xr);
      Fq three = Fq::one();
      three = add(add(three, three), Fq::one());
      const Fq rhs = add(mul(sqr(x), x), three);
      // y = rhs^((q + 1) / 4), most significant bit first
      Fq y = Fq::one();
#pragma unroll 1
      for (int bit = 253; bit >= 0; bit--) {
        y = sqr(y);
        if ((exponent.v[bit >> 5] >> (bit & 31)) & 1u) y = mul(y, rhs);
      }
      if (sqr(y) != rhs) {
        ok = false;  // x^3 + 3 is not a square: no such point
      } else {
        const Fq yc = from_mont(y);
        uint32_t neg_y[8];
        (void)sub8(neg_y, m, yc.v);
        const bool is_larger = gt256(yc.v, neg_y);
        if (is_larger != flag_neg) y = sub(Fq::zero(), y);
        p.x = x;
        p.y = y;
      }
    }
    if (!ok) atomicMax(bad, (unsigned long long)i + 1);
    out[i] = p;
  }
}

}  // namespace

extern "C" {

int zk_g1_compress(zk_ctx* ctx, const uint64_t* affine, zk_mem affine_mem, uint64_t n, uint8_t* out, zk_mem out_mem) {
  if (!ctx || (n && (!affine || !out))) return fail(ZK_ERR_ARG, "g1_compress: NULL argument");
  if (n == 0) return ZK_OK;
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  char* base = nullptr;
  const size_t in_b = affine_mem == ZK_MEM_HOST ? n * sizeof(Affine) : 0, out_b = out_mem == ZK_MEM_HOST ? n * 32 : 0;
  int rc = ctx->reserve_work(in_b + out_b + 1024, (void**)&base);
  if (rc) return rc;
  const Affine* d_in = reinterpret_cast<const Affine*>(affine);
  if (affine_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, affine, in_b, cudaMemcpyHostToDevice, s));
    d_in = reinterpret_cast<const Affine*>(base);
  }
  uint4* d_out = out_mem == ZK_MEM_HOST ? reinterpret_cast<uint4*>(base + ((in_b + 255) & ~(size_t)255)) : reinterpret_cast<uint4*>(out);
  uint64_t blocks = (n + 127) / 128;
  if (blocks > (uint64_t)ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  k_g1_compress<<<(unsigned)blocks, 128, 0, s>>>(d_in, n, d_out);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, n * 32, cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_g1_decompress(zk_ctx* ctx, const uint8_t* in, zk_mem in_mem, uint64_t n, uint64_t* affine_out, zk_mem out_mem) {
  if (!ctx || (n && (!in || !affine_out))) return fail(ZK_ERR_ARG, "g1_decompress: NULL argument");
  if (n == 0) return ZK_OK;
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  char* base = nullptr;
  const size_t in_b = in_mem == ZK_MEM_HOST ? n * 32 : 0, out_b = out_mem == ZK_MEM_HOST ? n * sizeof(Affine) : 0;
  int rc = ctx->reserve_work(256 + ((in_b + 255) & ~(size_t)255) + out_b + 1024, (void**)&base);
  if (rc) return rc;
  unsigned long long* d_bad = reinterpret_cast<unsigned long long*>(base);
  ZK_CUDA(cudaMemsetAsync(d_bad, 0, 8, s));
  const uint4* d_in = reinterpret_cast<const uint4*>(in);
  if (in_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base + 256, in, in_b, cudaMemcpyHostToDevice, s));
    d_in = reinterpret_cast<const uint4*>(base + 256);
  }
  Affine* d_out = out_mem == ZK_MEM_HOST ? reinterpret_cast<Affine*>(base + 256 + ((in_b + 255) & ~(size_t)255))
                                         : reinterpret_cast<Affine*>(affine_out);
  // (q + 1) / 4
  Limbs8 e;
  uint64_t carry = 1;
  for (int k = 0; k < 8; k++) {
    const uint64_t t = (uint64_t)FqParams::mod(k) + carry;
    e.v[k] = (uint32_t)t;
    carry = t >> 32;
  }
  for (int k = 0; k < 8; k++) e.v[k] = (e.v[k] >> 2) | (k < 7 ? e.v[k + 1] << 30 : 0u);
  uint64_t blocks = (n + 127) / 128;
  if (blocks > (uint64_t)ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  k_g1_decompress<<<(unsigned)blocks, 128, 0, s>>>(d_in, n, e, d_out, d_bad);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, d_bad, 8, cudaMemcpyDeviceToHost, s));
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(affine_out, d_out, n * sizeof(Affine), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  unsigned long long bad = 0;
  memcpy(&bad, ctx->host_small, 8);
  if (bad) return fail(ZK_ERR_ARG, "g1_decompress: encoding %llu is not a point (flags, x >= q, or x^3 + 3 not a square)", bad - 1);
  return ZK_OK;
}

}  // extern "C"
