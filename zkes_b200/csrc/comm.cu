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

// ---- exchange of the round messages through peer memory (the protocol: internal.hpp, ExchangeBox)
// One single-block kernel per rank and exchange, for the rounds that the host steps: stores this
// rank's partial sums into every rank's box, waits (bounded) for the others' in its own box, adds
// them in rank order and publishes the complete message to the polling host.  When the wait runs
// out the kernel reports through the error word beside the host's sequence word and returns.
__global__ void __launch_bounds__(256) k_exchange_sum(const Fr* vals, int n_vals, const PeerExchange px, unsigned int xseq,
                                                      Fr* out, const MsgSink sink, unsigned int* pub_error) {
  __shared__ uint32_t stage[kPeerRanks * kPeerVals * 8];
  __shared__ Fr v[kPeerVals];
  __shared__ int ok_shared;
  const int t = threadIdx.x;
  if (t < n_vals) v[t] = vals[t];
  __syncthreads();
  const bool ok = peer_exchange_sum(px, xseq, v, n_vals, stage, &ok_shared, t, blockDim.x);
  if (t < n_vals && ok) {
    out[t] = v[t];
    if (sink.pub_flag) st_fr_sys(sink.pub_msg + t, v[t]);
  }
  if (sink.pub_flag) {
    if (t == 0) *reinterpret_cast<volatile unsigned int*>(pub_error) = ok ? 0u : 1u;
    __threadfence_system();
    __syncthreads();
    if (t == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag) = sink.seq;
  }
}

// Block r stores this rank's chunks into rank r's box, fences, raises its flag there, then waits for
// rank r's flag in this rank's own box: when the kernel ends, every chunk has arrived here.
__global__ void __launch_bounds__(256) k_peer_gather(const PeerExchange px, unsigned int gseq, int n_tables, uint32_t m,
                                                     const Fr* t0, const Fr* t1, const Fr* t2, const Fr* t3,
                                                     unsigned int* error_word) {
  const int r = blockIdx.x;
  ExchangeBox* theirs = px.peers.box[r];
  const Fr* src[kMaxPolys] = {t0, t1, t2, t3};
  const uint32_t chunks = m * 2;  // 16-byte pieces per table chunk
  for (int i = 0; i < n_tables; i++) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src[i]);
    uint4* d4 = reinterpret_cast<uint4*>(&theirs->gather[i][(size_t)px.rank * m]);
    for (uint32_t k = threadIdx.x; k < chunks; k += blockDim.x) d4[k] = s4[k];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile unsigned int*>(&theirs->gather_flag[px.rank]) = gseq;
    const volatile unsigned int* f = reinterpret_cast<const volatile unsigned int*>(&px.peers.box[px.rank]->gather_flag[r]);
    unsigned int polls = 0;
    while (*f != gseq) {
      if (++polls > px.spin_limit) {
        atomicExch(error_word, 3u);
        break;
      }
      __nanosleep(64);
    }
    __threadfence_system();
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
  unsigned int gseq = 0;       // table hand-overs so far
  bool poisoned = false;       // a sharded call failed: the ranks' counters may differ, nothing more runs on it
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
  // all-gather (handle, ok) through NCCL: 128 bytes per rank.  The staging is the communicator's own gather
  // buffer (512 bytes per rank, allocated before this function runs): a rank never skips a collective because
  // of a local failure, it takes part and carries the failure in its ok byte, so that all ranks agree.
  constexpr size_t kRec = 128;
  static_assert(sizeof(cudaIpcMemHandle_t) < kRec, "record too small");
  static_assert(kRec * 2 <= 16 * sizeof(Fr), "the gather buffer holds a record per rank and this rank's own");
  unsigned char* d_rec = reinterpret_cast<unsigned char*>(c->gather_buf);
  std::vector<unsigned char> rec(kRec * (c->world + 1), 0);
  memcpy(rec.data(), &handle, sizeof handle);
  rec[kRec - 1] = mine_ok;
  bool good = cudaMemcpyAsync(d_rec, rec.data(), kRec, cudaMemcpyHostToDevice, s) == cudaSuccess &&
              g_nccl.all_gather(d_rec, d_rec + kRec, kRec, 1, c->comm, s) == 0 &&
              cudaMemcpyAsync(rec.data() + kRec, d_rec + kRec, kRec * c->world, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
              cudaStreamSynchronize(s) == cudaSuccess;
  if (!good) cudaGetLastError();
  bool all_ok = good;
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
  std::vector<unsigned char> oks(kRec * (c->world + 1), 0);
  oks[0] = open_ok;
  good = cudaMemcpyAsync(d_rec, oks.data(), kRec, cudaMemcpyHostToDevice, s) == cudaSuccess &&
         g_nccl.all_gather(d_rec, d_rec + kRec, kRec, 1, c->comm, s) == 0 &&
         cudaMemcpyAsync(oks.data() + kRec, d_rec + kRec, kRec * c->world, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
         cudaStreamSynchronize(s) == cudaSuccess;
  if (!good) {
    cudaGetLastError();
    return;
  }
  bool every = true;
  for (int r = 0; r < c->world; r++) every = every && oks[kRec * (r + 1)] == 1;
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
bool comm_poisoned(const zk_comm* c) { return c && c->poisoned; }
void comm_poison(zk_comm* c) {
  if (c) c->poisoned = true;
}

// Arguments for kernels that exchange through the peer boxes themselves; false when the ranks have
// no peer mapping (or the option is off) and the caller has to stay on the host-stepped exchange.
bool comm_peer_args(const zk_ctx* ctx, const zk_comm* c, PeerExchange* out) {
  if (!c || c->world == 1 || !c->peer_ok || !ctx->peer_exchange) return false;
  out->peers = c->peers;
  out->rank = c->rank;
  out->world = c->world;
  out->xseq_base = c->xseq;
  // a poll is a load from this GPU's memory plus a 32 ns pause, about a microsecond: 16 s and more by default.
  // The ranks of a prove are separate host processes and may reach a call seconds apart (one still copying its
  // inputs); the bound is there to end a wait for a rank that is gone, not to police that skew
  out->spin_limit = ctx->exchange_wait_ms * 1024u;
  return true;
}
// Every rank's m-entry chunk of each of the n_tables tables, gathered in rank order into this rank's
// box by the ranks' own stores; tables_out[i] is the complete table i (kGatherEntries = world * m
// entries at most).  error_word (device) is set to 3 when a wait ran out.
int comm_peer_gather(zk_ctx* ctx, zk_comm* c, int n_tables, const Fr* const* chunks, uint32_t m, unsigned int* error_word,
                     const Fr** tables_out) {
  PeerExchange px;
  if (!comm_peer_args(ctx, c, &px)) return fail(ZK_ERR_COMM, "peer gather without a peer mapping");
  if (n_tables > kMaxPolys || (uint64_t)m * c->world > kGatherEntries) return fail(ZK_ERR_ARG, "peer gather: too large");
  c->gseq++;
  const Fr* t[kMaxPolys] = {nullptr, nullptr, nullptr, nullptr};
  for (int i = 0; i < n_tables; i++) t[i] = chunks[i];
  k_peer_gather<<<c->world, 256, 0, ctx->stream>>>(px, c->gseq, n_tables, m, t[0], t[1], t[2], t[3], error_word);
  ctx->launches++;
  for (int i = 0; i < n_tables; i++) tables_out[i] = c->box->gather[i];
  return ZK_OK;
}
// Accounts for `n` exchanges a kernel made on its own.
void comm_peer_advance(zk_comm* c, unsigned int n) { c->xseq += n; }
int comm_rank(const zk_comm* c) { return c ? c->rank : 0; }

// vals (device, n_vals <= 16 elements) <- element-wise sum over all ranks; stream-ordered.
int comm_sum_fr(zk_ctx* ctx, zk_comm* c, Fr* vals, int n_vals) {
  if (!c || c->world == 1) return ZK_OK;
  if (c->peer_ok && ctx->peer_exchange && n_vals <= kPeerVals) {
    PeerExchange px;
    comm_peer_args(ctx, c, &px);
    c->xseq++;
    unsigned int* pub_error = ctx->rs.sink.pub_flag ? ctx->rs.sink.pub_flag + 1 : nullptr;
    k_exchange_sum<<<1, 256, 0, ctx->stream>>>(vals, n_vals, px, c->xseq, vals, ctx->rs.sink, pub_error);
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
  CtxLock lk(ctx, true);
  ctx = lk.lane;
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

int zk_comm_wait_selftest(zk_ctx* ctx, uint32_t polls) {
  if (!ctx || polls == 0 || polls > (1u << 22)) return fail(ZK_ERR_ARG, "comm_wait_selftest: polls must be in 1 .. 2^22");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  ExchangeBox* box = nullptr;
  cudaError_t e = cudaMalloc(&box, sizeof(ExchangeBox));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ZK_ERR_OOM, "comm_wait_selftest: %s", cudaGetErrorString(e));
  }
  ZK_CUDA(cudaMemsetAsync(box, 0, sizeof(ExchangeBox), s));
  // two ranks on paper, one in fact: both boxes are this one, so rank 0's own words arrive and rank 1's never do
  PeerExchange px;
  for (int r = 0; r < kPeerRanks; r++) px.peers.box[r] = r < 2 ? box : nullptr;
  px.rank = 0;
  px.world = 2;
  px.xseq_base = 0;
  px.spin_limit = polls;
  RoundScratch sc = ctx->next_msg_scratch(false);
  volatile unsigned int* flag =
      reinterpret_cast<volatile unsigned int*>(reinterpret_cast<char*>(ctx->mailbox) + 16 * sizeof(Fr));
  k_exchange_sum<<<1, 256, 0, s>>>(ctx->rs.sink.msg, 3, px, 1u, ctx->rs.sink.msg, sc.sink, sc.sink.pub_flag + 1);
  ctx->launches++;
  cudaError_t le = cudaGetLastError();
  cudaError_t se = cudaStreamSynchronize(s);
  cudaFree(box);
  if (le != cudaSuccess || se != cudaSuccess) return fail(ZK_ERR_CUDA, "comm_wait_selftest: %s", cudaGetErrorString(le != cudaSuccess ? le : se));
  const bool published = flag[0] == sc.sink.seq, timed_out = flag[1] != 0;
  flag[1] = 0;  // the error word belongs to the next exchange again
  if (!published) return fail(ZK_ERR_CUDA, "comm_wait_selftest: the kernel did not publish");
  if (timed_out) return fail(ZK_ERR_TIMEOUT, "comm_wait_selftest: the wait for rank 1 ran out after %u polls (expected)", polls);
  return ZK_OK;
}

void zk_comm_free(zk_ctx* ctx, zk_comm* c) {
  if (!c) return;
  if (ctx) {
    CtxLock lk(ctx, true);
  ctx = lk.lane;
    cudaStreamSynchronize(ctx->stream);
    peer_teardown(c);
    cudaFree(c->gather_buf);
    if (c->comm && g_nccl.destroy) g_nccl.destroy(c->comm);
  }
  delete c;
}

}  // extern "C"
