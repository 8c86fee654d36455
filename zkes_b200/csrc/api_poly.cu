// C ABI: eq tables and fix_variables_from_right.
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace zk {
// Builds eq(., point) in `table` (device, 2^k elements); `point_dev` is device scratch for k elements.
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table) {
  cudaStream_t s = ctx->stream;
  if (k) ZK_CUDA(cudaMemcpyAsync(point_dev, point_host, (size_t)k * sizeof(Fr), cudaMemcpyHostToDevice, s));
  ctx->prof_begin(ZK_PROF_FROM_RIGHT, 32.0 * 3 * (double)(1ull << k), 1);
  ctx->launches += launch_eq_table(point_dev, reinterpret_cast<const Fr*>(point_host), k, table, ctx->sm_count, s);
  ctx->prof_end();
  return ZK_OK;
}

// out_dev[lo] = sum_hi eq(point)[hi] f[hi * 2^(n-k) + lo]; f_dev holds 2^n elements on the device.
// scratch must hold k + 2^k + splits * 2^(n-k) elements.
size_t from_right_scratch_elems(zk_ctx* ctx, uint32_t n, uint32_t k) {
  const uint64_t lo_n = 1ull << (n - k), hi_n = 1ull << k;
  return (size_t)k + 8 + hi_n + (size_t)from_right_splits(lo_n, hi_n, ctx->sm_count) * lo_n;
}
int fix_from_right_device(zk_ctx* ctx, uint32_t n, const Fr* f_dev, uint32_t k, const uint64_t* point_host, Fr* scratch,
                          Fr* out_dev) {
  const uint64_t lo_n = 1ull << (n - k), hi_n = 1ull << k;
  Fr* point_dev = scratch;
  Fr* eq = scratch + k + 8;
  Fr* partial = eq + hi_n;
  int rc = eq_table_device(ctx, point_host, k, point_dev, eq);
  if (rc) return rc;
  ctx->prof_begin(ZK_PROF_FROM_RIGHT, 32.0 * (double)((1ull << n) + lo_n), 1);
  ctx->launches += launch_from_right(f_dev, eq, lo_n, hi_n, partial, out_dev, ctx->sm_count, ctx->stream);
  ctx->prof_end();
  ZK_CUDA(cudaGetLastError());
  return ZK_OK;
}
}  // namespace zk

extern "C" {

int zk_eq_table(zk_ctx* ctx, uint32_t k, const uint64_t* point, uint64_t* out, zk_mem out_mem) {
  if (!ctx || !out || (k && !point)) return fail(ZK_ERR_ARG, "eq_table: NULL argument");
  if (k > 34) return fail(ZK_ERR_ARG, "eq_table: k %u too large", k);
  CtxLock lk(ctx);
  ctx = lk.lane;
  const uint64_t size = 1ull << k;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((k + 8 + (out_mem == ZK_MEM_HOST ? size : 0)) * sizeof(Fr), (void**)&base);
  if (rc) return rc;
  Fr* table = out_mem == ZK_MEM_HOST ? base + k + 8 : reinterpret_cast<Fr*>(out);
  rc = eq_table_device(ctx, point, k, base, table);
  if (rc) return rc;
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, table, size * sizeof(Fr), cudaMemcpyDeviceToHost, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZK_OK;
}

int zk_weighted_fold_from_right(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k,
                                const uint64_t* weights, zk_mem weights_mem, uint64_t* out, zk_mem out_mem) {
  if (!ctx || !evals || !out || !weights) return fail(ZK_ERR_ARG, "weighted_fold_from_right: NULL argument");
  if (k > n || n > 34) return fail(ZK_ERR_ARG, "weighted_fold_from_right: bad dimensions");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << n, lo_n = 1ull << (n - k), hi_n = 1ull << k;
  const size_t in_elems = evals_mem == ZK_MEM_HOST ? size : 0;
  const size_t w_elems = weights_mem == ZK_MEM_HOST ? hi_n : 0;
  const size_t out_elems = out_mem == ZK_MEM_HOST ? lo_n : 0;
  const size_t part = (size_t)from_right_splits(lo_n, hi_n, ctx->sm_count) * lo_n;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((in_elems + w_elems + out_elems + part + 16) * sizeof(Fr), (void**)&base);
  if (rc) return rc;
  const Fr* f = reinterpret_cast<const Fr*>(evals);
  const Fr* w = reinterpret_cast<const Fr*>(weights);
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, evals, size * sizeof(Fr), cudaMemcpyHostToDevice, s));
    f = base;
  }
  if (weights_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base + in_elems, weights, hi_n * sizeof(Fr), cudaMemcpyHostToDevice, s));
    w = base + in_elems;
  }
  Fr* d_out = out_mem == ZK_MEM_HOST ? base + in_elems + w_elems : reinterpret_cast<Fr*>(out);
  ctx->launches += launch_from_right(f, w, lo_n, hi_n, base + in_elems + w_elems + out_elems, d_out, ctx->sm_count, s);
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, lo_n * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_mle_eval(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, const uint64_t* point, uint64_t* out) {
  if (!ctx || !evals || !out || (n && !point)) return fail(ZK_ERR_ARG, "mle_eval: NULL argument");
  if (n > 34) return fail(ZK_ERR_ARG, "mle_eval: n %u too large", n);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << n;
  const size_t in_elems = evals_mem == ZK_MEM_HOST ? size : 0;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((in_elems + size + n + 16) * sizeof(Fr), (void**)&base);
  if (rc) return rc;
  const Fr* f = reinterpret_cast<const Fr*>(evals);
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, evals, size * sizeof(Fr), cudaMemcpyHostToDevice, s));
    f = base;
  }
  Fr* eq = base + in_elems;
  rc = eq_table_device(ctx, point, n, eq + size, eq);
  if (rc) return rc;
  RoundScratch sc = ctx->rs;
  sc.sink.pub_flag = nullptr;  // read back with a copy: nothing polls this result
  launch_dot(f, eq, size, sc, s);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->rs.sink.msg, sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  memcpy(out, ctx->host_small, sizeof(Fr));
  return ZK_OK;
}

int zk_fix_from_right(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k, const uint64_t* point,
                      uint64_t* out, zk_mem out_mem) {
  if (!ctx || !evals || !out || (k && !point)) return fail(ZK_ERR_ARG, "fix_from_right: NULL argument");
  if (k > n) return fail(ZK_ERR_ARG, "invalid size of partial point");
  if (n > 34) return fail(ZK_ERR_ARG, "fix_from_right: n %u too large", n);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << n, lo_n = 1ull << (n - k);
  const size_t in_elems = evals_mem == ZK_MEM_HOST ? size : 0;
  const size_t out_elems = out_mem == ZK_MEM_HOST ? lo_n : 0;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((in_elems + out_elems + from_right_scratch_elems(ctx, n, k) + 16) * sizeof(Fr), (void**)&base);
  if (rc) return rc;
  const Fr* f = reinterpret_cast<const Fr*>(evals);
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, evals, size * sizeof(Fr), cudaMemcpyHostToDevice, s));
    f = base;
  }
  Fr* d_out = out_mem == ZK_MEM_HOST ? base + in_elems : reinterpret_cast<Fr*>(out);
  if (k == 0) {
    ZK_CUDA(cudaMemcpyAsync(d_out, f, size * sizeof(Fr), cudaMemcpyDeviceToDevice, s));
  } else {
    rc = fix_from_right_device(ctx, n, f, k, point, base + in_elems + out_elems, d_out);
    if (rc) return rc;
  }
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, lo_n * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

}  // extern "C"
