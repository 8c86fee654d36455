// C ABI: KZH commit / open of sparse polynomials (non-zero entries given as (index, value) pairs):
// sparse_kzh2_commit / open (src/crypto/polycommit/sparse_kzh2.rs:14-127) and sparse_kzh3_commit / open
// (sparse_kzh3.rs:32-232).  Commit is two gather-MSMs (sparse_msm, polycommit/mod.rs:10-31): one over
// the full vector, one with every entry routed to the row of its x index.  The opens are in api_kzh.cu.
#include "../../include/zkb200.h"
#include "kzh.hpp"

#include <vector>

using namespace zk;

namespace zk {
int normalize_device(zk_ctx* ctx, const Jacobian* in, uint64_t n, Affine* out);
// keyset.cu: distinct keys in increasing order through a bitmap of the domain
size_t keyset_scratch_bytes(uint32_t n_terms, uint32_t num_var);
int keyset_order(zk_ctx* ctx, const uint64_t* positions_dev, const uint64_t* term_begin_dev, uint32_t n_terms, uint64_t total,
                 uint32_t num_var, void* scratch, uint32_t* keys_out, uint32_t bad_host[2]);
}

namespace {

inline size_t al(size_t x) { return (x + 255) & ~(size_t)255; }

__global__ void k_split_index(const uint64_t* __restrict__ idx, uint32_t n, uint32_t low_bits, uint64_t limit,
                              uint32_t* full, uint32_t* low, uint32_t* row, uint32_t* bad) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint64_t v = idx[i];
    if (v >= limit) *bad = 1;
    full[i] = (uint32_t)v;
    low[i] = (uint32_t)(v & ((1ull << low_bits) - 1));
    row[i] = (uint32_t)(v >> low_bits);
  }
}

}  // namespace

extern "C" {

int zk_sparse_kzh_commit(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                         uint64_t* c_affine_out, uint64_t* d_x_jac_out) {
  if (!ctx || !srs || !c_affine_out || !d_x_jac_out || (nnz && !indices))
    return fail(ZK_ERR_ARG, "sparse_kzh_commit: NULL argument");
  if (srs->world != 1) return fail(ZK_ERR_ARG, "sparse_kzh_commit: needs an unsharded SRS");
  if (nnz >> 31) return fail(ZK_ERR_ARG, "sparse_kzh_commit: too many entries");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint64_t rows = 1ull << srs->x_log;
  const uint32_t low_bits = srs->n - srs->x_log;
  char* base = nullptr;
  const bool selection = !vals && nnz && srs->n <= 30;  // every listed entry is one
  int rc = ctx->reserve_work(al(nnz * 8) + al(nnz * sizeof(Fr)) + 3 * al(nnz * 4 + 4) + al((rows + 1) * sizeof(Jacobian)) +
                             al(sizeof(Affine)) + al(rows * sizeof(Xyzz)) + 256 +
                             (selection ? al(keyset_scratch_bytes(1, srs->n)) : 0) + 1024, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  uint64_t* d_idx = (uint64_t*)take(nnz * 8);
  Fr* d_val = (Fr*)take(nnz * sizeof(Fr));
  uint32_t* d_full = (uint32_t*)take(nnz * 4 + 4);
  uint32_t* d_low = (uint32_t*)take(nnz * 4 + 4);
  uint32_t* d_row = (uint32_t*)take(nnz * 4 + 4);
  Jacobian* d_jac = (Jacobian*)take((rows + 1) * sizeof(Jacobian));
  Affine* d_c = (Affine*)take(sizeof(Affine));
  void* d_sel = take(rows * sizeof(Xyzz));
  uint64_t* d_begin = (uint64_t*)take(16);
  uint32_t* bad = ctx->rs.sink.counter + 16;
  if (selection) {
    // A selection polynomial: both commitments are plain sums of SRS points.  The indices are put in order through
    // a bitmap of the domain (they are distinct: a duplicate sends the call to the general path below, which adds
    // the point twice as the reference's loop would); a row of d_x is then a contiguous run of the list, and the
    // digit, sort and bucket passes of the general MSM are not needed.
    void* ks = take(keyset_scratch_bytes(1, srs->n));
    uint64_t* h_begin = reinterpret_cast<uint64_t*>(reinterpret_cast<char*>(ctx->host_small) + 2048);
    h_begin[0] = 0;
    h_begin[1] = nnz;
    ZK_CUDA(cudaMemcpyAsync(d_idx, indices, nnz * 8, cudaMemcpyHostToDevice, st));
    ZK_CUDA(cudaMemcpyAsync(d_begin, h_begin, 16, cudaMemcpyHostToDevice, st));
    uint32_t bad_keys[2] = {0, 0};
    rc = keyset_order(ctx, d_idx, d_begin, 1, nnz, srs->n, ks, d_full, bad_keys);
    if (rc) return rc;
    if (bad_keys[0]) return fail(ZK_ERR_ARG, "sparse_kzh_commit: an index is outside the SRS domain");
    if (!bad_keys[1]) {
      rc = msm_select_sums(ctx, srs->h[0], srs->h[1], d_full, (uint32_t)nnz, low_bits, (uint32_t)rows, d_jac, d_sel);
      if (rc) return rc;
      Jacobian* h_c = reinterpret_cast<Jacobian*>(reinterpret_cast<char*>(ctx->host_small) + 4096);
      ZK_CUDA(cudaMemcpyAsync(h_c, d_jac + rows, sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
      ZK_CUDA(cudaMemcpyAsync(d_x_jac_out, d_jac, rows * sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
      ZK_CUDA(cudaStreamSynchronize(st));
      const Affine c_aff = jacobian_to_affine_host(*h_c);
      memcpy(c_affine_out, &c_aff, sizeof(Affine));
      return ZK_OK;
    }
  }
  if (nnz) {
    ZK_CUDA(cudaMemcpyAsync(d_idx, indices, nnz * 8, cudaMemcpyHostToDevice, st));
    if (vals) {
      ZK_CUDA(cudaMemcpyAsync(d_val, vals, nnz * sizeof(Fr), cudaMemcpyHostToDevice, st));
    } else {  // a selection polynomial: every listed entry is one
      launch_fill_ones(d_val, (uint32_t)nnz, ctx->sm_count, st);
      ctx->launches++;
    }
    ZK_CUDA(cudaMemsetAsync(bad, 0, 4, st));
    k_split_index<<<ctx->sm_count * 4, 256, 0, st>>>(d_idx, (uint32_t)nnz, low_bits, 1ull << srs->n, d_full, d_low, d_row, bad);
    ctx->launches++;
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, bad, 4, cudaMemcpyDeviceToHost, st));
    ZK_CUDA(cudaStreamSynchronize(st));
    uint32_t b = 0;
    memcpy(&b, ctx->host_small, 4);
    if (b) return fail(ZK_ERR_ARG, "sparse_kzh_commit: an index is outside the SRS domain");
  }
  // C = sparse_msm(h_full, indices, scalars)   (sparse_kzh2.rs:27-38, sparse_kzh3.rs:45-56)
  rc = msm_run(ctx, srs->h[0], d_full, d_val, nnz, 1, d_jac + rows, &ctx->last_msm);
  if (rc) return rc;
  // d_x[x] = sparse_msm(h_mid, low indices of the entries with that x, their values)   (sparse_kzh2.rs:42-80)
  rc = msm_run_rows(ctx, srs->h[1], d_low, d_row, d_val, nnz, (uint32_t)rows, d_jac, nullptr);
  if (rc) return rc;
  Jacobian* h_c = reinterpret_cast<Jacobian*>(reinterpret_cast<char*>(ctx->host_small) + 4096);
  ZK_CUDA(cudaMemcpyAsync(h_c, d_jac + rows, sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(d_x_jac_out, d_jac, rows * sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  const Affine c_aff = jacobian_to_affine_host(*h_c);  // the commitment's affine form (into_affine)
  memcpy(c_affine_out, &c_aff, sizeof(Affine));
  return ZK_OK;
}

}  // extern "C"
