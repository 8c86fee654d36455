// C ABI: the table steps of Einsum::prove ahead of its sumcheck (variable permutation, integer-table fold).
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace {
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
}  // namespace

namespace zk {
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table);
}

extern "C" {

int zk_permute_by_ranges(zk_ctx* ctx, uint32_t n, uint32_t elem_bytes, const void* evals, zk_mem evals_mem,
                         uint32_t n_ranges, const uint64_t* ranges, void* out, zk_mem out_mem) {
  if (!ctx || !evals || !out || !ranges) return fail(ZK_ERR_ARG, "permute_by_ranges: NULL argument");
  if (elem_bytes != 16 && elem_bytes != 32) return fail(ZK_ERR_ARG, "permute_by_ranges: elements of 16 or 32 bytes");
  if (n > 34) return fail(ZK_ERR_ARG, "permute_by_ranges: n %u too large", n);
  if (n_ranges == 0) return fail(ZK_ERR_ARG, "ranges must not be empty");
  if (n_ranges > 40) return fail(ZK_ERR_ARG, "permute_by_ranges: at most 40 ranges");
  // the reference's checks (einsum.rs:143-161): valid ranges that cover every variable exactly once
  uint64_t seen = 0;
  uint32_t covered = 0;
  uint32_t r32[80];
  for (uint32_t r = 0; r < n_ranges; r++) {
    const uint64_t start = ranges[2 * r], end = ranges[2 * r + 1];
    if (!(start <= end && end <= n)) return fail(ZK_ERR_ARG, "invalid range (%llu, %llu)", (unsigned long long)start, (unsigned long long)end);
    for (uint64_t v = start; v < end; v++) {
      if (seen & (1ull << v)) return fail(ZK_ERR_ARG, "variable %llu appears in multiple ranges", (unsigned long long)v);
      seen |= 1ull << v;
      covered++;
    }
    r32[2 * r] = (uint32_t)start;
    r32[2 * r + 1] = (uint32_t)end;
  }
  if (covered != n) return fail(ZK_ERR_ARG, "ranges must cover all variables exactly once");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t bytes = (1ull << n) * elem_bytes;
  const size_t in_b = evals_mem == ZK_MEM_HOST ? align_up(bytes, 256) : 0, out_b = out_mem == ZK_MEM_HOST ? align_up(bytes, 256) : 0;
  char* base = nullptr;
  int rc = ctx->reserve_work(in_b + out_b + 256, (void**)&base);
  if (rc) return rc;
  const void* d_in = evals;
  void* d_out = out;
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, evals, bytes, cudaMemcpyHostToDevice, s));
    d_in = base;
  }
  if (out_mem == ZK_MEM_HOST) d_out = base + in_b;
  if (d_in == d_out) return fail(ZK_ERR_ARG, "permute_by_ranges: in-place permutation is not supported");
  ctx->launches += launch_permute_ranges(d_in, d_out, n, elem_bytes, r32, n_ranges, ctx->sm_count, s);
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, bytes, cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_fix_variables_int(zk_ctx* ctx, uint32_t num_vars, const void* t, zk_mem t_mem, uint32_t k, const uint64_t* point,
                         uint64_t* out, zk_mem out_mem) {
  if (!ctx || !t || !out || (k && !point)) return fail(ZK_ERR_ARG, "fix_variables_int: NULL argument");
  if (k > num_vars) return fail(ZK_ERR_ARG, "fix_variables_int: %u challenges for %u variables", k, num_vars);
  if (num_vars > 34) return fail(ZK_ERR_ARG, "fix_variables_int: num_vars %u too large", num_vars);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t n_rows = 1ull << k, m_cols = 1ull << (num_vars - k);
  const uint64_t in_bytes = (1ull << num_vars) * 16;
  const uint32_t splits = n_rows >= 32 ? int_fold_splits(n_rows, m_cols, ctx->sm_count) : 1;
  const size_t in_b = t_mem == ZK_MEM_HOST ? align_up(in_bytes, 256) : 0;
  const size_t out_elems = out_mem == ZK_MEM_HOST ? m_cols : 0;
  const size_t part_elems = splits > 1 ? (size_t)splits * m_cols : 0;
  char* base = nullptr;
  int rc = ctx->reserve_work(in_b + (n_rows + k + 16 + out_elems + part_elems) * sizeof(Fr) + 256, (void**)&base);
  if (rc) return rc;
  const void* d_t = t;
  if (t_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, t, in_bytes, cudaMemcpyHostToDevice, s));
    d_t = base;
  }
  Fr* eq = reinterpret_cast<Fr*>(base + in_b);
  Fr* pt_dev = eq + n_rows;
  Fr* d_out = out_mem == ZK_MEM_HOST ? pt_dev + k + 16 : reinterpret_cast<Fr*>(out);
  Fr* partial = pt_dev + k + 16 + out_elems;
  rc = eq_table_device(ctx, point, k, pt_dev, eq);
  if (rc) return rc;
  ctx->prof_begin(ZK_PROF_OTHER, 16.0 * (double)(1ull << num_vars) + 32.0 * (double)m_cols, 1);
  ctx->launches += launch_int_fold(d_t, eq, n_rows, m_cols, partial, d_out, ctx->sm_count, s);
  ctx->prof_end();
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, m_cols * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

}  // extern "C"
