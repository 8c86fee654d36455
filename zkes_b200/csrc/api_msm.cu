// C ABI: multi-scalar multiplications over G1 and point normalisation.
#include "../../include/zkb200.h"
#include "msm.hpp"

using namespace zk;

namespace {

__global__ void k_normalize(const Jacobian* __restrict__ in, uint64_t n, Affine* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const Jacobian j = in[i];
    Affine a;
    if (j.z.is_zero()) {
      a.x = Fq::zero();
      a.y = Fq::zero();
    } else {
      const Fq zi = inverse(j.z), zi2 = sqr(zi);
      a.x = mul(j.x, zi2);
      a.y = mul(j.y, mul(zi2, zi));
    }
    out[i] = a;
  }
}

}  // namespace

namespace zk {
// out[i] = affine form of in[i]; device pointers.
int normalize_device(zk_ctx* ctx, const Jacobian* in, uint64_t n, Affine* out) {
  if (n == 0) return 0;
  uint64_t blocks = (n + 127) / 128;
  if (blocks > (uint64_t)ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  k_normalize<<<(unsigned)blocks, 128, 0, ctx->stream>>>(in, n, out);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  return 0;
}
}  // namespace zk

namespace {

// Shared driver: stage host inputs in the work scratch, run, copy the Jacobian rows out.
int msm_entry(zk_ctx* ctx, const uint64_t* bases, zk_mem bases_mem, uint64_t n_bases, const uint64_t* indices,
              const uint64_t* scalars, zk_mem scalars_mem, uint64_t n, uint64_t rows, uint64_t* out_jac, zk_mem out_mem,
              const char* who) {
  if (!ctx || !out_jac) return fail(ZK_ERR_ARG, "%s: NULL argument", who);
  if (n && (!bases || !scalars)) return fail(ZK_ERR_ARG, "%s: NULL input", who);
  if (rows == 0) return ZK_OK;
  if (rows >= (1ull << 31) || n >= (1ull << 31)) return fail(ZK_ERR_ARG, "%s: dimensions too large", who);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  size_t need = 4096 + rows * sizeof(Jacobian) + 256;
  if (bases_mem == ZK_MEM_HOST) need += n_bases * sizeof(Affine) + 256;
  if (scalars_mem == ZK_MEM_HOST) need += n * rows * sizeof(Fr) + 256;
  if (indices) need += n * (4 + 8) + 512;
  char* base = nullptr;
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += (bytes + 255) & ~(size_t)255; return p; };
  Jacobian* d_out = (Jacobian*)take(rows * sizeof(Jacobian));
  const Affine* d_bases = (const Affine*)bases;
  if (bases_mem == ZK_MEM_HOST && n_bases) {
    Affine* p = (Affine*)take(n_bases * sizeof(Affine));
    ZK_CUDA(cudaMemcpyAsync(p, bases, n_bases * sizeof(Affine), cudaMemcpyHostToDevice, s));
    d_bases = p;
  }
  const Fr* d_scalars = (const Fr*)scalars;
  if (scalars_mem == ZK_MEM_HOST && n) {
    Fr* p = (Fr*)take(n * rows * sizeof(Fr));
    ZK_CUDA(cudaMemcpyAsync(p, scalars, n * rows * sizeof(Fr), cudaMemcpyHostToDevice, s));
    d_scalars = p;
  }
  uint32_t* d_gather = nullptr;
  if (indices && n) {  // indices follow the scalars' memory kind
    uint64_t* i64 = (uint64_t*)take(n * 8);
    d_gather = (uint32_t*)take(n * 4);
    ZK_CUDA(cudaMemcpyAsync(i64, indices, n * 8, cudaMemcpyDefault, s));
    ZK_CUDA(cudaMemsetAsync(ctx->rs.sink.counter + 16, 0, 4, s));
    launch_narrow_idx(i64, (uint32_t)n, d_gather, ctx->rs.sink.counter + 16, ctx->sm_count, s);
    launch_check_bound(d_gather, (uint32_t)n, n_bases, ctx->rs.sink.counter + 16, ctx->sm_count, s);
    ctx->launches += 2;
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->rs.sink.counter + 16, 4, cudaMemcpyDeviceToHost, s));
    ZK_CUDA(cudaStreamSynchronize(s));
    uint32_t bad = 0;
    memcpy(&bad, ctx->host_small, 4);
    if (bad) return fail(ZK_ERR_ARG, "%s: an index is out of range of the base table", who);
  }
  ctx->prof_begin(ZK_PROF_MSM, 0.0, 8);
  rc = msm_run(ctx, d_bases, d_gather, d_scalars, n, (uint32_t)rows, d_out, &ctx->last_msm);
  ctx->prof_end();
  if (rc) return rc;
  ZK_CUDA(cudaMemcpyAsync(out_jac, d_out, rows * sizeof(Jacobian), cudaMemcpyDefault, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  (void)out_mem;
  return ZK_OK;
}

}  // namespace

extern "C" {

int zk_msm_g1(zk_ctx* ctx, const uint64_t* bases, zk_mem bases_mem, const uint64_t* scalars, zk_mem scalars_mem,
              uint64_t n, uint64_t* out_jac, zk_mem out_mem) {
  return msm_entry(ctx, bases, bases_mem, n, nullptr, scalars, scalars_mem, n, 1, out_jac, out_mem, "msm_g1");
}

int zk_msm_g1_batched(zk_ctx* ctx, const uint64_t* bases, zk_mem bases_mem, uint64_t n_bases, const uint64_t* scalars,
                      zk_mem scalars_mem, uint64_t n_rows, uint64_t* out_jac, zk_mem out_mem) {
  return msm_entry(ctx, bases, bases_mem, n_bases, nullptr, scalars, scalars_mem, n_bases, n_rows, out_jac, out_mem,
                   "msm_g1_batched");
}

int zk_msm_g1_gather(zk_ctx* ctx, const uint64_t* all_bases, zk_mem bases_mem, uint64_t n_bases, const uint64_t* indices,
                     const uint64_t* scalars, zk_mem scalars_mem, uint64_t k, uint64_t* out_jac, zk_mem out_mem) {
  if (k && !indices) return fail(ZK_ERR_ARG, "msm_g1_gather: NULL indices");
  return msm_entry(ctx, all_bases, bases_mem, n_bases, k ? indices : nullptr, scalars, scalars_mem, k, 1, out_jac, out_mem,
                   "msm_g1_gather");
}

int zk_g1_normalize(zk_ctx* ctx, const uint64_t* jac, zk_mem jac_mem, uint64_t n, uint64_t* affine_out, zk_mem out_mem) {
  if (!ctx || (n && (!jac || !affine_out))) return fail(ZK_ERR_ARG, "g1_normalize: NULL argument");
  if (n == 0) return ZK_OK;
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  char* base = nullptr;
  int rc = ctx->reserve_work(n * (sizeof(Jacobian) + sizeof(Affine)) + 1024, (void**)&base);
  if (rc) return rc;
  const Jacobian* d_in = (const Jacobian*)jac;
  if (jac_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, jac, n * sizeof(Jacobian), cudaMemcpyHostToDevice, s));
    d_in = (const Jacobian*)base;
  }
  Affine* d_out = out_mem == ZK_MEM_DEVICE ? (Affine*)affine_out
                                           : (Affine*)(base + ((n * sizeof(Jacobian) + 255) & ~(size_t)255));
  uint64_t blocks = (n + 127) / 128;
  if (blocks > (uint64_t)ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  k_normalize<<<(unsigned)blocks, 128, 0, s>>>(d_in, n, d_out);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(affine_out, d_out, n * sizeof(Affine), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_msm_work(zk_ctx* ctx, uint64_t* calls, uint64_t* entries, uint64_t* buckets, int reset) {
  if (!ctx) return fail(ZK_ERR_ARG, "msm_work: NULL context");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  uint64_t c = ctx->msm_calls, e = ctx->msm_entries_sum, b = ctx->msm_bucket_sum;
  for (zk_ctx* l : ctx->lanes) {  // lanes at rest: a caller reads this between its calls
    c += l->msm_calls;
    e += l->msm_entries_sum;
    b += l->msm_bucket_sum;
    if (reset) l->msm_calls = l->msm_entries_sum = l->msm_bucket_sum = 0;
  }
  if (calls) *calls = c;
  if (entries) *entries = e;
  if (buckets) *buckets = b;
  if (reset) ctx->msm_calls = ctx->msm_entries_sum = ctx->msm_bucket_sum = 0;
  return ZK_OK;
}

int zk_msm_last_stats(zk_ctx* ctx, int* window_bits, int* windows, int* max_bits, uint64_t* entries, uint64_t* buckets) {
  if (!ctx) return fail(ZK_ERR_ARG, "msm_last_stats: NULL context");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  if (window_bits) *window_bits = ctx->last_msm.window_bits;
  if (windows) *windows = ctx->last_msm.windows;
  if (max_bits) *max_bits = ctx->last_msm.max_bits;
  if (entries) *entries = ctx->last_msm.entries;
  if (buckets) *buckets = ctx->last_msm.buckets;
  return ZK_OK;
}

}  // extern "C"
