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
#include <vector>

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

// ---- exchange of the round messages through peer memory
//
// Every rank owns one ExchangeBox in its own HBM and holds a peer mapping of every other rank's
// box.  A round's exchange is one single-block kernel per rank: it stores this rank's partial sums
// into slot [rank] of every rank's box (ordinary stores over NVLink), fences, stores the exchange's
// sequence number into the matching flag of every box, then polls the flags of its *own* box until
// all ranks' values of this exchange have landed, adds them in rank order (the same order on every
// rank, so the sums are bit-identical) and publishes the complete message to the polling host.
// Ranks only ever write remotely and read locally.  Two sets of slots alternate: a rank can be at
// most one exchange ahead of the slowest, because finishing exchange k needs everybody's flag k.
// The wait is bounded; when it runs out the kernel reports through the error word and returns.
__global__ void __launch_bounds__(256) k_exchange_sum(const Fr* vals, int n_vals, int rank, int world, const PeerTable peers,
                                                      unsigned int xseq, unsigned int spin_limit, Fr* out,
                                                      const MsgSink sink, unsigned int* pub_error) {
  __shared__ int ok;
  const int par = xseq & 1u, t = threadIdx.x;
  if (t == 0) ok = 1;
  if (t < world * n_vals) {
    const int r = t / n_vals, c = t - r * n_vals;
    st_fr_sys(&peers.box[r]->slots[par][rank][c], vals[c]);
  }
  __threadfence_system();
  __syncthreads();
  if (t < world) *reinterpret_cast<volatile unsigned int*>(&peers.box[t]->flags[par][rank]) = xseq;
  ExchangeBox* mine = peers.box[rank];
  if (t < world) {
    const volatile unsigned int* f = reinterpret_cast<const volatile unsigned int*>(&mine->flags[par][t]);
    unsigned int polls = 0;
    while (*f != xseq) {
      if (++polls > spin_limit) {
        ok = 0;
        break;
      }
      __nanosleep(32);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (t < n_vals && ok) {
    Fr sum = Fr::zero();
    for (int r = 0; r < world; r++) {
      const volatile uint32_t* q = reinterpret_cast<const volatile uint32_t*>(&mine->slots[par][r][t]);
      Fr v;
#pragma unroll
      for (int i = 0; i < 8; i++) v.v[i] = q[i];
      sum = add(sum, v);
    }
    out[t] = sum;
    if (sink.pub_flag) st_fr_sys(sink.pub_msg + t, sum);
  }
  if (sink.pub_flag) {
    if (t == 0) *reinterpret_cast<volatile unsigned int*>(pub_error) = ok ? 0u : 1u;
    __threadfence_system();
    __syncthreads();
    if (t == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag) = sink.seq;
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
  // exchange through peer memory (all ranks agree on peer_ok)
  bool peer_ok = false;
  ExchangeBox* box = nullptr;  // this rank's box
  PeerTable peers;             // every rank's box as this rank addresses it
  unsigned int xseq = 0;       // exchanges so far: the same on every rank
};

// Maps every rank's exchange box into this process.  Leaves c->peer_ok false (and the NCCL path
// in use) when any rank could not: the ranks agree on the outcome through one more all-gather.
static void peer_setup(zk_ctx* ctx, zk_comm* c) {
  for (int r = 0; r < kPeerRanks; r++) c->peers.box[r] = nullptr;
  if (c->world > kPeerRanks) return;
  cudaStream_t s = ctx->stream;
  unsigned char mine_ok = 1;
  cudaIpcMemHandle_t handle;
  memset(&handle, 0, sizeof handle);
  if (cudaMalloc(&c->box, sizeof(ExchangeBox)) != cudaSuccess) {
    cudaGetLastError();
    c->box = nullptr;
    mine_ok = 0;
  } else {
    cudaMemsetAsync(c->box, 0, sizeof(ExchangeBox), s);
    if (cudaIpcGetMemHandle(&handle, c->box) != cudaSuccess) {
      cudaGetLastError();
      mine_ok = 0;
    }
  }
  // all-gather (handle, ok) through NCCL: 128 bytes per rank
  constexpr size_t kRec = 128;
  static_assert(sizeof(cudaIpcMemHandle_t) < kRec, "record too small");
  unsigned char* d_rec = nullptr;
  if (cudaMalloc(&d_rec, kRec * (c->world + 1)) != cudaSuccess) {
    cudaGetLastError();
    return;  // cannot even exchange the outcome; every rank that fails here stays on NCCL, the others time out loudly
  }
  std::vector<unsigned char> rec(kRec * (c->world + 1), 0);
  memcpy(rec.data(), &handle, sizeof handle);
  rec[kRec - 1] = mine_ok;
  bool good = cudaMemcpyAsync(d_rec, rec.data(), kRec, cudaMemcpyHostToDevice, s) == cudaSuccess &&
              g_nccl.all_gather(d_rec, d_rec + kRec, kRec, 1, c->comm, s) == 0 &&
              cudaMemcpyAsync(rec.data() + kRec, d_rec + kRec, kRec * c->world, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
              cudaStreamSynchronize(s) == cudaSuccess;
  cudaFree(d_rec);
  if (!good) {
    cudaGetLastError();
    return;
  }
  bool all_ok = true;
  for (int r = 0; r < c->world; r++) all_ok = all_ok && rec[kRec * (r + 1) + kRec - 1] == 1;
  unsigned char open_ok = all_ok ? 1 : 0;
  if (all_ok) {
    for (int r = 0; r < c->world; r++) {
      if (r == c->rank) {
        c->peers.box[r] = c->box;
        continue;
      }
      cudaIpcMemHandle_t h;
      memcpy(&h, rec.data() + kRec * (r + 1), sizeof h);
      void* p = nullptr;
      if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        open_ok = 0;
        break;
      }
      c->peers.box[r] = reinterpret_cast<ExchangeBox*>(p);
    }
  }
  // second agreement: every rank opened every box
  unsigned char* d_ok = nullptr;
  if (cudaMalloc(&d_ok, 256 * (c->world + 1)) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  std::vector<unsigned char> oks(256 * (c->world + 1), 0);
  oks[0] = open_ok;
  good = cudaMemcpyAsync(d_ok, oks.data(), 256, cudaMemcpyHostToDevice, s) == cudaSuccess &&
         g_nccl.all_gather(d_ok, d_ok + 256, 256, 1, c->comm, s) == 0 &&
         cudaMemcpyAsync(oks.data() + 256, d_ok + 256, 256 * c->world, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
         cudaStreamSynchronize(s) == cudaSuccess;
  cudaFree(d_ok);
  if (!good) {
    cudaGetLastError();
    return;
  }
  bool every = true;
  for (int r = 0; r < c->world; r++) every = every && oks[256 * (r + 1)] == 1;
  c->peer_ok = every;
}

static void peer_teardown(zk_comm* c) {
  for (int r = 0; r < c->world && r < kPeerRanks; r++)
    if (r != c->rank && c->peers.box[r]) cudaIpcCloseMemHandle(c->peers.box[r]);
  if (c->box) cudaFree(c->box);
  cudaGetLastError();
}

namespace zk {
int comm_world(const zk_comm* c) { return c ? c->world : 1; }

// Arguments for kernels that exchange through the peer boxes themselves; false when the ranks have
// no peer mapping (or the option is off) and the caller has to stay on the host-stepped exchange.
bool comm_peer_args(const zk_ctx* ctx, const zk_comm* c, PeerExchange* out) {
  if (!c || c->world == 1 || !c->peer_ok || !ctx->peer_exchange) return false;
  out->peers = c->peers;
  out->rank = c->rank;
  out->world = c->world;
  out->xseq_base = c->xseq;
  out->spin_limit = 40u << 20;
  return true;
}
// Accounts for `n` exchanges a kernel made on its own.
void comm_peer_advance(zk_comm* c, unsigned int n) { c->xseq += n; }
int comm_rank(const zk_comm* c) { return c ? c->rank : 0; }

// vals (device, n_vals <= 16 elements) <- element-wise sum over all ranks; stream-ordered.
int comm_sum_fr(zk_ctx* ctx, zk_comm* c, Fr* vals, int n_vals) {
  if (!c || c->world == 1) return ZK_OK;
  if (c->peer_ok && ctx->peer_exchange && n_vals <= kPeerVals) {
    c->xseq++;
    unsigned int* pub_error = ctx->rs.sink.pub_flag ? ctx->rs.sink.pub_flag + 1 : nullptr;
    // polls pause 32 ns: the limit is a few seconds, far beyond the skew between ranks of a healthy run
    k_exchange_sum<<<1, 256, 0, ctx->stream>>>(vals, n_vals, c->rank, c->world, c->peers, c->xseq, 40u << 20, vals,
                                               ctx->rs.sink, pub_error);
    ctx->launches++;
    return ZK_OK;
  }
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
  if (world > 1) peer_setup(ctx, c);
  *out = c;
  return ZK_OK;
}

int zk_comm_peer_exchange(const zk_comm* c) { return c && c->peer_ok ? 1 : 0; }

void zk_comm_free(zk_ctx* ctx, zk_comm* c) {
  if (!c) return;
  if (ctx) {
    CtxLock lk(ctx);
    cudaStreamSynchronize(ctx->stream);
    peer_teardown(c);
    cudaFree(c->gather_buf);
    if (c->comm && g_nccl.destroy) g_nccl.destroy(c->comm);
  }
  delete c;
}

}  // extern "C"
