// Multi-GPU exchange: one process per GPU, NCCL all-gather of the per-round partial sums.
//
// NCCL is bound at run time (dlopen of libnccl.so.2: the copy the host process already loaded,
// e.g. PyTorch's, or the system one) so the library has no link-time dependency on it.  The
// host distributes the unique id (torch.distributed broadcast, MPI, a file ...).
#include "../../include/zkb200.h"
#include "ctx.hpp"
#include "reduce.cuh"
#include "ec.cuh"

#include <dlfcn.h>

using namespace zk;

namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclId { char internal[128]; };
typedef int (*fn_get_id)(NcclId*);
typedef int (*fn_init_rank)(ncclComm_t*, int, NcclId, int);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t);
typedef int (*fn_destroy)(ncclComm_t);
typedef const char* (*fn_errstr)(int);

struct NcclApi {
  void* handle = nullptr;
  fn_get_id get_id = nullptr;
  fn_init_rank init_rank = nullptr;
  fn_all_gather all_gather = nullptr;
  fn_destroy destroy = nullptr;
  fn_errstr errstr = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl.handle) return ZK_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return fail(ZK_ERR_COMM, "NCCL not found: %s", dlerror());
  NcclApi a;
  a.handle = h;
  a.get_id = (fn_get_id)dlsym(h, "ncclGetUniqueId");
  a.init_rank = (fn_init_rank)dlsym(h, "ncclCommInitRank");
  a.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
  a.destroy = (fn_destroy)dlsym(h, "ncclCommDestroy");
  a.errstr = (fn_errstr)dlsym(h, "ncclGetErrorString");
  if (!a.get_id || !a.init_rank || !a.all_gather || !a.destroy) return fail(ZK_ERR_COMM, "NCCL symbols missing");
  g_nccl = a;
  return ZK_OK;
}

// out[c] = sum over ranks of gathered[rank * n_vals + c]
// The sum is the complete round message: it is also published to the polling host.
__global__ void k_sum_ranks(const Fr* __restrict__ gathered, int world, int n_vals, Fr* out, const MsgSink sink) {
  const int c = threadIdx.x;
  if (c < n_vals) {
    Fr s = gathered[c];
    for (int r = 1; r < world; r++) s = add(s, gathered[r * n_vals + c]);
    out[c] = s;
    if (sink.pub_flag) st_fr_sys(sink.pub_msg + c, s);
  }
  if (sink.pub_flag) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag) = sink.seq;
  }
}

// point <- sum of `world` Jacobian points (rank-major in gathered)
__global__ void k_sum_points(const Jacobian* __restrict__ gathered, int world, int n_points, Jacobian* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_points) return;
  Xyzz acc = Xyzz::inf();
  for (int r = 0; r < world; r++) {
    const Jacobian j = gathered[(size_t)r * n_points + i];
    if (j.z.is_zero()) continue;
    Xyzz p;
    p.x = j.x;
    p.y = j.y;
    p.zz = sqr(j.z);
    p.zzz = mul(p.zz, j.z);
    acc = add(acc, p);
  }
  out[i] = to_jacobian(acc);
}

// vals[i] <- sum over ranks of gathered[r * n + i]
__global__ void k_sum_ranks_vec(const Fr* __restrict__ gathered, int world, uint64_t n, Fr* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    Fr s = gathered[i];
    for (int r = 1; r < world; r++) s = add(s, gathered[(uint64_t)r * n + i]);
    out[i] = s;
  }
}

}  // namespace

struct zk_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  Fr* gather_buf = nullptr;  // world * 16 elements
};

namespace zk {
int comm_world(const zk_comm* c) { return c ? c->world : 1; }
int comm_rank(const zk_comm* c) { return c ? c->rank : 0; }

// vals (device, n_vals <= 16 elements) <- element-wise sum over all ranks; stream-ordered.
int comm_sum_fr(zk_ctx* ctx, zk_comm* c, Fr* vals, int n_vals) {
  if (!c || c->world == 1) return ZK_OK;
  int rc = g_nccl.all_gather(vals, c->gather_buf, (size_t)n_vals * sizeof(Fr), 1 /*ncclUint8*/, c->comm, ctx->stream);
  if (rc != 0) return fail(ZK_ERR_COMM, "ncclAllGather: %s", g_nccl.errstr ? g_nccl.errstr(rc) : "error");
  k_sum_ranks<<<1, 32, 0, ctx->stream>>>(c->gather_buf, c->world, n_vals, vals, ctx->rs.sink);
  ctx->launches++;
  return ZK_OK;
}

// out (device, world * n_vals elements, rank-major) <- every rank's vals; stream-ordered.
int comm_gather_fr(zk_ctx* ctx, zk_comm* c, const Fr* vals, int n_vals, Fr* out) {
  if (!c || c->world == 1) {
    ZK_CUDA(cudaMemcpyAsync(out, vals, (size_t)n_vals * sizeof(Fr), cudaMemcpyDeviceToDevice, ctx->stream));
    return ZK_OK;
  }
  int rc = g_nccl.all_gather(vals, out, (size_t)n_vals * sizeof(Fr), 1, c->comm, ctx->stream);
  if (rc != 0) return fail(ZK_ERR_COMM, "ncclAllGather: %s", g_nccl.errstr ? g_nccl.errstr(rc) : "error");
  return ZK_OK;
}

// point[0 .. n_points) (device) <- element-wise group sum over all ranks; uses the aux scratch.
int comm_sum_points_n(zk_ctx* ctx, zk_comm* c, Jacobian* points, int n_points) {
  if (!c || c->world == 1) return ZK_OK;
  void* buf = nullptr;
  int rc = ctx->reserve_aux((size_t)c->world * n_points * sizeof(Jacobian) + 256, &buf);
  if (rc) return rc;
  rc = comm_gather_bytes(ctx, c, points, (size_t)n_points * sizeof(Jacobian), buf);
  if (rc) return rc;
  k_sum_points<<<(n_points + 63) / 64, 64, 0, ctx->stream>>>((const Jacobian*)buf, c->world, n_points, points);
  ctx->launches++;
  return ZK_OK;
}
int comm_sum_points(zk_ctx* ctx, zk_comm* c, Jacobian* point) { return comm_sum_points_n(ctx, c, point, 1); }

// vals[0 .. n) (device) <- element-wise field sum over all ranks; uses the aux scratch.
int comm_sum_fr_vec(zk_ctx* ctx, zk_comm* c, Fr* vals, uint64_t n) {
  if (!c || c->world == 1 || n == 0) return ZK_OK;
  void* buf = nullptr;
  int rc = ctx->reserve_aux((size_t)c->world * n * sizeof(Fr) + 256, &buf);
  if (rc) return rc;
  rc = comm_gather_bytes(ctx, c, vals, n * sizeof(Fr), buf);
  if (rc) return rc;
  uint64_t blocks = (n + 255) / 256;
  if (blocks > (uint64_t)ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  k_sum_ranks_vec<<<(unsigned)blocks, 256, 0, ctx->stream>>>((const Fr*)buf, c->world, n, vals);
  ctx->launches++;
  return ZK_OK;
}

// Raw bytes (device buffers), for the MSM partial points.
int comm_gather_bytes(zk_ctx* ctx, zk_comm* c, const void* send, size_t bytes, void* recv) {
  if (!c || c->world == 1) {
    ZK_CUDA(cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return ZK_OK;
  }
  int rc = g_nccl.all_gather(send, recv, bytes, 1, c->comm, ctx->stream);
  if (rc != 0) return fail(ZK_ERR_COMM, "ncclAllGather: %s", g_nccl.errstr ? g_nccl.errstr(rc) : "error");
  return ZK_OK;
}
}  // namespace zk

extern "C" {

int zk_comm_unique_id(uint8_t out[128]) {
  if (!out) return fail(ZK_ERR_ARG, "comm_unique_id: NULL argument");
  int rc = load_nccl();
  if (rc) return rc;
  NcclId id;
  rc = g_nccl.get_id(&id);
  if (rc != 0) return fail(ZK_ERR_COMM, "ncclGetUniqueId failed (%d)", rc);
  memcpy(out, id.internal, 128);
  return ZK_OK;
}

int zk_comm_init(zk_ctx* ctx, int rank, int world, const uint8_t unique_id[128], zk_comm** out) {
  if (!ctx || !out || !unique_id) return fail(ZK_ERR_ARG, "comm_init: NULL argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(ZK_ERR_ARG, "comm_init: rank %d of %d", rank, world);
  if (world & (world - 1)) return fail(ZK_ERR_ARG, "comm_init: the number of ranks must be a power of two");
  int rc = load_nccl();
  if (rc) return rc;
  CtxLock lk(ctx);
  zk_comm* c = new zk_comm();
  c->rank = rank;
  c->world = world;
  NcclId id;
  memcpy(id.internal, unique_id, 128);
  rc = g_nccl.init_rank(&c->comm, world, id, rank);
  if (rc != 0) {
    delete c;
    return fail(ZK_ERR_COMM, "ncclCommInitRank: %s", g_nccl.errstr ? g_nccl.errstr(rc) : "error");
  }
  cudaError_t e = cudaMalloc(&c->gather_buf, (size_t)world * 16 * sizeof(Fr));
  if (e != cudaSuccess) {
    g_nccl.destroy(c->comm);
    delete c;
    return fail(ZK_ERR_OOM, "comm_init: %s", cudaGetErrorString(e));
  }
  *out = c;
  return ZK_OK;
}

void zk_comm_free(zk_ctx* ctx, zk_comm* c) {
  if (!c) return;
  if (ctx) {
    CtxLock lk(ctx);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(c->gather_buf);
    if (c->comm && g_nccl.destroy) g_nccl.destroy(c->comm);
  }
  delete c;
}

}  // extern "C"
