// C ABI: multi-GPU forms of the MSM and of KZH commit / open.  Points are sharded by contiguous
// range (for KZH: whole x-rows), every rank computes its partial result, and the partial G1
// sums (96 bytes each) or partial tables are all-gathered and added on every rank.
#include "../../include/zkb200.h"
#include "kzh.hpp"

#include <vector>

using namespace zk;

namespace zk {
int comm_sum_points_n(zk_ctx* ctx, zk_comm* c, Jacobian* points, int n_points);
int comm_sum_fr_vec(zk_ctx* ctx, zk_comm* c, Fr* vals, uint64_t n);
int normalize_device(zk_ctx* ctx, const Jacobian* in, uint64_t n, Affine* out);
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table);
}  // namespace zk

namespace {
inline size_t al(size_t x) { return (x + 255) & ~(size_t)255; }
}

extern "C" {

static int msm_g1_sharded_impl(zk_ctx* ctx, zk_comm* comm, const uint64_t* local_bases, zk_mem bases_mem,
                      const uint64_t* local_scalars, zk_mem scalars_mem, uint64_t n_local, uint64_t* out_jac) {
  if (!ctx || !comm || !out_jac) return fail(ZK_ERR_ARG, "msm_g1_sharded: NULL argument");
  if (n_local && (!local_bases || !local_scalars)) return fail(ZK_ERR_ARG, "msm_g1_sharded: NULL input");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  char* base = nullptr;
  size_t need = 4096 + al(sizeof(Jacobian));
  if (bases_mem == ZK_MEM_HOST) need += al(n_local * sizeof(Affine));
  if (scalars_mem == ZK_MEM_HOST) need += al(n_local * sizeof(Fr));
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  Jacobian* d_out = (Jacobian*)take(sizeof(Jacobian));
  const Affine* d_bases = (const Affine*)local_bases;
  const Fr* d_scalars = (const Fr*)local_scalars;
  if (bases_mem == ZK_MEM_HOST && n_local) {
    Affine* p = (Affine*)take(n_local * sizeof(Affine));
    ZK_CUDA(cudaMemcpyAsync(p, local_bases, n_local * sizeof(Affine), cudaMemcpyHostToDevice, s));
    d_bases = p;
  }
  if (scalars_mem == ZK_MEM_HOST && n_local) {
    Fr* p = (Fr*)take(n_local * sizeof(Fr));
    ZK_CUDA(cudaMemcpyAsync(p, local_scalars, n_local * sizeof(Fr), cudaMemcpyHostToDevice, s));
    d_scalars = p;
  }
  rc = msm_run(ctx, d_bases, nullptr, d_scalars, n_local, 1, d_out, &ctx->last_msm);
  if (rc) return rc;
  rc = comm_sum_points_n(ctx, comm, d_out, 1);
  if (rc) return rc;
  ZK_CUDA(cudaMemcpyAsync(out_jac, d_out, sizeof(Jacobian), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_msm_g1_sharded(zk_ctx* ctx, zk_comm* comm, const uint64_t* local_bases, zk_mem bases_mem,
                      const uint64_t* local_scalars, zk_mem scalars_mem, uint64_t n_local, uint64_t* out_jac) {
  if (!comm) return fail(ZK_ERR_ARG, "msm_g1_sharded: NULL communicator");
  return sharded_call(comm, "msm_g1_sharded", [&] { return msm_g1_sharded_impl(ctx, comm, local_bases, bases_mem, local_scalars, scalars_mem, n_local, out_jac); });
}

// Commit with an SRS made by zk_kzh_srs_setup_sharded: local_evals is this rank's slab of the
// polynomial (2^n / world elements = its x-rows).  Every rank receives c and the full d_x.
static int kzh_commit_sharded_impl(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals,
                          zk_mem evals_mem, uint64_t* c_affine_out, uint64_t* d_x_jac_out) {
  if (!ctx || !comm || !srs || !local_evals || !c_affine_out || !d_x_jac_out)
    return fail(ZK_ERR_ARG, "kzh_commit_sharded: NULL argument");
  if (comm_world(comm) != srs->world || comm_rank(comm) != srs->rank)
    return fail(ZK_ERR_ARG, "kzh_commit_sharded: the SRS was set up for rank %d of %d", srs->rank, srs->world);
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint64_t slab = srs->count[0], rows = 1ull << srs->x_log, rows_local = rows / srs->world;
  char* base = nullptr;
  int rc = ctx->reserve_work(al(slab * sizeof(Fr)) + al((rows + 1) * sizeof(Jacobian)) + al(sizeof(Affine)) + 1024, (void**)&base);
  if (rc) return rc;
  Fr* staging = reinterpret_cast<Fr*>(base);
  Jacobian* d_jac = reinterpret_cast<Jacobian*>(base + al(slab * sizeof(Fr)));  // [rows of d_x][C]
  Affine* d_c = reinterpret_cast<Affine*>(base + al(slab * sizeof(Fr)) + al((rows + 1) * sizeof(Jacobian)));
  const Fr* f = reinterpret_cast<const Fr*>(local_evals);
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(staging, local_evals, slab * sizeof(Fr), cudaMemcpyHostToDevice, st));
    f = staging;
  }
  // partial C over this rank's slab of h_full, then the group sum over ranks
  MsmPrep prep;  // one analysis pass over the scalars serves both MSMs
  rc = msm_run(ctx, srs->h[0], nullptr, f, slab, 1, d_jac + rows, &ctx->last_msm, &prep);
  if (rc) return rc;
  rc = comm_sum_points_n(ctx, comm, d_jac + rows, 1);
  if (rc) return rc;
  // this rank's rows of d_x, written at their place in the full vector, then all-gathered in place
  Jacobian* mine = d_jac + rows_local * srs->rank;
  rc = msm_run(ctx, srs->h[1], nullptr, f, srs->count[1], (uint32_t)rows_local, mine, nullptr, &prep);
  if (rc) return rc;
  void* tmp = nullptr;
  rc = ctx->reserve_aux(rows * sizeof(Jacobian) + 256, &tmp);
  if (rc) return rc;
  rc = comm_gather_bytes(ctx, comm, mine, rows_local * sizeof(Jacobian), tmp);
  if (rc) return rc;
  Jacobian* h_c = reinterpret_cast<Jacobian*>(reinterpret_cast<char*>(ctx->host_small) + 4096);
  ZK_CUDA(cudaMemcpyAsync(h_c, d_jac + rows, sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(d_x_jac_out, tmp, rows * sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  const Affine c_aff = jacobian_to_affine_host(*h_c);  // the commitment's affine form (into_affine)
  memcpy(c_affine_out, &c_aff, sizeof(Affine));
  return ZK_OK;
}

int zk_kzh_commit_sharded(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals,
                          zk_mem evals_mem, uint64_t* c_affine_out, uint64_t* d_x_jac_out) {
  if (!comm) return fail(ZK_ERR_ARG, "kzh_commit_sharded: NULL communicator");
  return sharded_call(comm, "kzh_commit_sharded", [&] { return kzh_commit_sharded_impl(ctx, comm, srs, local_evals, evals_mem, c_affine_out, d_x_jac_out); });
}

// fix_variables_from_right over a table sharded on its top variables: local_evals holds the
// rank's 2^n / world entries; point binds the k highest variables (k >= log2 world).  Every rank
// receives the full 2^(n-k) result.
static int fix_from_right_sharded_impl(zk_ctx* ctx, zk_comm* comm, uint32_t n, const uint64_t* local_evals, zk_mem evals_mem,
                              uint32_t k, const uint64_t* point, uint64_t* out) {
  if (!ctx || !comm || !local_evals || !out || (k && !point)) return fail(ZK_ERR_ARG, "fix_from_right_sharded: NULL argument");
  const int world = comm_world(comm), rank = comm_rank(comm);
  uint32_t logw = 0;
  while ((1 << logw) < world) logw++;
  if (k > n || k < logw) return fail(ZK_ERR_ARG, "fix_from_right_sharded: k = %u must cover the %u sharded variables", k, logw);
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t lo_n = 1ull << (n - k), hi_n = 1ull << k, hi_local = hi_n / world, slab = hi_local * lo_n;
  const uint32_t splits = from_right_splits(lo_n, hi_local, ctx->sm_count);
  char* base = nullptr;
  size_t need = al((k + 8) * sizeof(Fr)) + al(hi_n * sizeof(Fr)) + al((size_t)splits * lo_n * sizeof(Fr)) + al(lo_n * sizeof(Fr)) + 1024;
  if (evals_mem == ZK_MEM_HOST) need += al(slab * sizeof(Fr));
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  Fr* pt_dev = (Fr*)take((k + 8) * sizeof(Fr));
  Fr* eq = (Fr*)take(hi_n * sizeof(Fr));
  Fr* partial = (Fr*)take((size_t)splits * lo_n * sizeof(Fr));
  Fr* d_out = (Fr*)take(lo_n * sizeof(Fr));
  const Fr* f = reinterpret_cast<const Fr*>(local_evals);
  if (evals_mem == ZK_MEM_HOST) {
    Fr* p = (Fr*)take(slab * sizeof(Fr));
    ZK_CUDA(cudaMemcpyAsync(p, local_evals, slab * sizeof(Fr), cudaMemcpyHostToDevice, s));
    f = p;
  }
  rc = eq_table_device(ctx, point, k, pt_dev, eq);
  if (rc) return rc;
  // this rank's share: sum over its hi range with the matching slice of the eq table
  ctx->launches += launch_from_right(f, eq + hi_local * rank, lo_n, hi_local, partial, d_out, ctx->sm_count, s);
  rc = comm_sum_fr_vec(ctx, comm, d_out, lo_n);
  if (rc) return rc;
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(out, d_out, lo_n * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

int zk_fix_from_right_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t n, const uint64_t* local_evals, zk_mem evals_mem,
                              uint32_t k, const uint64_t* point, uint64_t* out) {
  if (!comm) return fail(ZK_ERR_ARG, "fix_from_right_sharded: NULL communicator");
  return sharded_call(comm, "fix_from_right_sharded", [&] { return fix_from_right_sharded_impl(ctx, comm, n, local_evals, evals_mem, k, point, out); });
}

}  // extern "C"
