// Seeded synthetic inputs generated on the device (benchmark and test data, not part of the
// proving path).  The stream is ChaCha20 (RFC 8439 block function, zero nonce) keyed by
// (seed, stream id); block i of the stream defines element i:
//   uniform Fr  : the 64 keystream bytes as a little-endian 512-bit integer, reduced mod r
//   small ints  : keystream word 0 reduced to a signed `bits`-bit integer, negatives as r - |v|
// so any range of elements can be produced independently by any number of threads.
#include "../../include/zkb200.h"
#include "ctx.hpp"
#include "reduce.cuh"

using namespace zk;

namespace {

__device__ __forceinline__ uint32_t rotl32(uint32_t v, int n) { return (v << n) | (v >> (32 - n)); }

__device__ __forceinline__ void chacha_block(uint64_t seed, uint64_t stream, uint32_t counter, uint32_t (&out)[16]) {
  uint32_t st[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u,
                     (uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)stream, (uint32_t)(stream >> 32),
                     0, 0, 0, 0, counter, 0, 0, 0};
  uint32_t x[16];
#pragma unroll
  for (int i = 0; i < 16; i++) x[i] = st[i];
#define ZK_QR(a, b, c, d)                 \
  x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 16); \
  x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 12); \
  x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 8);  \
  x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 7);
  for (int r = 0; r < 10; r++) {
    ZK_QR(0, 4, 8, 12) ZK_QR(1, 5, 9, 13) ZK_QR(2, 6, 10, 14) ZK_QR(3, 7, 11, 15)
    ZK_QR(0, 5, 10, 15) ZK_QR(1, 6, 11, 12) ZK_QR(2, 7, 8, 13) ZK_QR(3, 4, 9, 14)
  }
#undef ZK_QR
#pragma unroll
  for (int i = 0; i < 16; i++) out[i] = x[i] + st[i];
}

__global__ void k_gen_uniform(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, Fr* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t ks[16];
    chacha_block(seed, stream, (uint32_t)(start + i), ks);
    Fr lo, hi;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      lo.v[k] = ks[k];
      hi.v[k] = ks[8 + k];
    }
    // (lo + 2^256 hi) mod r in Montgomery form: lo * R + hi * R^2 = mont(R^2, lo) + mont(R^3, hi)
    const Fr v = add(mul(Fr::r2(), lo), mul(Fr::r3(), hi));
    uint4 a, b;
    fr_to_chunks(v, a, b);
    reinterpret_cast<uint4*>(out + i)[0] = a;
    reinterpret_cast<uint4*>(out + i)[1] = b;
  }
}

__global__ void k_gen_small(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int bits, Fr* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t ks[16];
    chacha_block(seed, stream, (uint32_t)(start + i), ks);
    const uint32_t u = ks[0] & ((1u << bits) - 1u);
    const int32_t sv = (int32_t)u - (int32_t)(1u << (bits - 1));  // [-2^(bits-1), 2^(bits-1))
    Fr c = Fr::zero();
    c.v[0] = (uint32_t)(sv < 0 ? -sv : sv);
    Fr v = to_mont(c);
    if (sv < 0) v = neg(v);
    uint4 a, b;
    fr_to_chunks(v, a, b);
    reinterpret_cast<uint4*>(out + i)[0] = a;
    reinterpret_cast<uint4*>(out + i)[1] = b;
  }
}

// round(N(0,1) * 2^scale_log2) from a Box-Muller transform of two keystream words, clamped to int16.
__global__ void k_gen_gauss(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int scale_log2, Fr* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t ks[16];
    chacha_block(seed, stream, (uint32_t)(start + i), ks);
    const double u1 = ((double)ks[0] + 1.0) / 4294967297.0, u2 = (double)ks[1] / 4294967296.0;
    double z = sqrt(-2.0 * log(u1)) * cospi(2.0 * u2) * (double)(1 << scale_log2);
    z = rint(z);
    if (z > 32767.0) z = 32767.0;
    if (z < -32767.0) z = -32767.0;
    const int32_t sv = (int32_t)z;
    Fr c = Fr::zero();
    c.v[0] = (uint32_t)(sv < 0 ? -sv : sv);
    Fr v = to_mont(c);
    if (sv < 0) v = neg(v);
    uint4 a, b;
    fr_to_chunks(v, a, b);
    reinterpret_cast<uint4*>(out + i)[0] = a;
    reinterpret_cast<uint4*>(out + i)[1] = b;
  }
}

}  // namespace

extern "C" int zk_gen_gauss_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int scale_log2,
                               uint64_t* out_dev) {
  if (!ctx || !out_dev) return fail(ZK_ERR_ARG, "gen_gauss_fr: NULL argument");
  if (scale_log2 < 0 || scale_log2 > 14) return fail(ZK_ERR_ARG, "gen_gauss_fr: scale_log2 must be in [0, 14]");
  if (start + count > (1ull << 32)) return fail(ZK_ERR_ARG, "gen_gauss_fr: the block counter is 32 bits");
  CtxLock lk(ctx);
  ctx = lk.lane;
  if (count) {
    k_gen_gauss<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(seed, stream, start, count, scale_log2, reinterpret_cast<Fr*>(out_dev));
    ctx->launches++;
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZK_OK;
}

extern "C" int zk_gen_uniform_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count,
                                 uint64_t* out_dev) {
  if (!ctx || !out_dev) return fail(ZK_ERR_ARG, "gen_uniform_fr: NULL argument");
  if (start + count > (1ull << 32)) return fail(ZK_ERR_ARG, "gen_uniform_fr: the block counter is 32 bits");
  CtxLock lk(ctx);
  ctx = lk.lane;
  if (count) {
    k_gen_uniform<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(seed, stream, start, count, reinterpret_cast<Fr*>(out_dev));
    ctx->launches++;
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZK_OK;
}

extern "C" int zk_gen_small_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int bits,
                               uint64_t* out_dev) {
  if (!ctx || !out_dev) return fail(ZK_ERR_ARG, "gen_small_fr: NULL argument");
  if (bits < 2 || bits > 31) return fail(ZK_ERR_ARG, "gen_small_fr: bits must be in [2, 31]");
  if (start + count > (1ull << 32)) return fail(ZK_ERR_ARG, "gen_small_fr: the block counter is 32 bits");
  CtxLock lk(ctx);
  ctx = lk.lane;
  if (count) {
    k_gen_small<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(seed, stream, start, count, bits, reinterpret_cast<Fr*>(out_dev));
    ctx->launches++;
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZK_OK;
}
