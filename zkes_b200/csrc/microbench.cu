// Dependency-light throughput probes used as roofline denominators for the integer-bound
// kernels: the 32-bit multiply-add rate (the nominal integer peak), wide multiply-adds inside carry
// chains (the form big-integer arithmetic needs), and the Montgomery product itself.
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace {

__global__ void k_imad(uint32_t* out, uint32_t b, uint32_t c, int iters) {
  uint32_t a[8];
#pragma unroll
  for (int k = 0; k < 8; k++) a[k] = threadIdx.x + k;
  for (int i = 0; i < iters; i++) {
#pragma unroll
    for (int k = 0; k < 8; k++) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(a[k]) : "r"(b), "r"(c));
  }
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < 8; k++) s ^= a[k];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

// Four independent madwide4 chains per thread (the Montgomery product's row primitive).
__global__ void k_chain(uint32_t* out, uint32_t b, int iters) {
  uint32_t acc[4][8];
#pragma unroll
  for (int c = 0; c < 4; c++)
#pragma unroll
    for (int k = 0; k < 8; k++) acc[c][k] = threadIdx.x * 97u + c * 8 + k;
  uint32_t x0 = threadIdx.x | 1u, x1 = x0 * 3u, x2 = x0 * 5u, x3 = x0 * 7u, cs = 0;
  for (int i = 0; i < iters; i++) {
#pragma unroll
    for (int c = 0; c < 4; c++) {
      madwide4(acc[c], x0, x1, x2, x3, b);
    }
  }
  uint32_t s = cs;
#pragma unroll
  for (int c = 0; c < 4; c++)
#pragma unroll
    for (int k = 0; k < 8; k++) s ^= acc[c][k];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

template <class P>
__global__ void k_modmul(Fp<P>* out, int iters) {
  Fp<P> x = Fp<P>::one(), y = Fp<P>::r2();
  x.v[0] ^= threadIdx.x;
  y.v[1] ^= blockIdx.x;
  Fp<P> z = Fp<P>::r3();
  for (int i = 0; i < iters; i++) {
    x = mul(x, y);
    z = mul(z, y);  // two independent chains per thread
  }
  out[blockIdx.x * blockDim.x + threadIdx.x] = add(x, z);
}

}  // namespace

extern "C" int zk_microbench(zk_ctx* ctx, int kind, int blocks, int threads, int iters, float* ms_out,
                             double* ops_out) {
  if (!ctx || !ms_out || !ops_out) return fail(ZK_ERR_ARG, "zk_microbench: NULL argument");
  if (blocks <= 0 || threads <= 0 || threads > 1024 || iters <= 0) return fail(ZK_ERR_ARG, "zk_microbench: bad launch shape");
  CtxLock lk(ctx);
  ctx = lk.lane;
  void* buf = nullptr;
  int rc = ctx->reserve_work((size_t)blocks * threads * 32, &buf);
  if (rc != ZK_OK) return rc;
  cudaEvent_t e0, e1;
  ZK_CUDA(cudaEventCreate(&e0));
  ZK_CUDA(cudaEventCreate(&e1));
  for (int rep = 0; rep < 2; rep++) {  // first repetition warms up
    ZK_CUDA(cudaEventRecord(e0, ctx->stream));
    switch (kind) {
      case 0: k_imad<<<blocks, threads, 0, ctx->stream>>>((uint32_t*)buf, 0x9e3779b9u, 12345u, iters); break;
      case 2: k_modmul<FrParams><<<blocks, threads, 0, ctx->stream>>>((Fr*)buf, iters); break;
      case 3: k_modmul<FqParams><<<blocks, threads, 0, ctx->stream>>>((Fq*)buf, iters); break;
      case 4: k_chain<<<blocks, threads, 0, ctx->stream>>>((uint32_t*)buf, 0x9e3779b9u, iters); break;
      default: return fail(ZK_ERR_ARG, "zk_microbench: unknown kind %d", kind);
    }
    ctx->launches++;
    ZK_CUDA(cudaEventRecord(e1, ctx->stream));
    ZK_CUDA(cudaEventSynchronize(e1));
    ZK_CUDA(cudaGetLastError());
  }
  ZK_CUDA(cudaEventElapsedTime(ms_out, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  // operations per thread: multiply-adds (0), Montgomery products (2, 3), wide multiply-adds inside carry chains (4)
  double per_thread = 8.0 * iters;
  if (kind == 2 || kind == 3) per_thread = 2.0 * iters;
  if (kind == 4) per_thread = 16.0 * iters;
  *ops_out = per_thread * blocks * (double)threads;
  return ZK_OK;
}
