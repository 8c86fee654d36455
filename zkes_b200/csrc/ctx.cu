#include "ctx.hpp"

using namespace zk;

int zk_ctx::setup() {
  ZK_CUDA(cudaSetDevice(device));
  ZK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  ZK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  ZK_CUDA(cudaStreamCreateWithFlags(&side_stream, cudaStreamNonBlocking));
  ZK_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
  ZK_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
  rs.max_blocks = sm_count * 8;
  rs.sm_count = sm_count;
  ZK_CUDA(cudaMalloc(&rs.sink.partials, sizeof(Fr) * (size_t)rs.max_blocks * (kMaxPolys + 1)));
  ZK_CUDA(cudaMalloc(&rs.sink.counter, 256));
  ZK_CUDA(cudaMemsetAsync(rs.sink.counter, 0, 256, stream));
  ZK_CUDA(cudaMalloc(&rs.sink.msg, sizeof(Fr) * 16));
  // host-mapped mailbox: 16 message elements, then the sequence word
  ZK_CUDA(cudaHostAlloc(&mailbox, 1024, cudaHostAllocMapped));
  memset(mailbox, 0, 1024);
  void* dev_view = nullptr;
  ZK_CUDA(cudaHostGetDevicePointer(&dev_view, mailbox, 0));
  rs.sink.pub_msg = reinterpret_cast<Fr*>(dev_view);
  rs.sink.pub_flag = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(dev_view) + 16 * sizeof(Fr));
  rs.sink.seq = 0;
  ZK_CUDA(cudaMalloc(&final_out, sizeof(Fr) * 16));
  ZK_CUDA(cudaMalloc(&tail_out, 8192));
  ZK_CUDA(cudaMalloc(&resident_sh, 8192));
  ZK_CUDA(cudaMemsetAsync(resident_sh, 0, 8192, stream));
  ZK_CUDA(cudaMalloc(&tail_buf, sizeof(Fr) * 64 * kMaxPolys * 4));
  ZK_CUDA(cudaHostAlloc(&host_small, 8192, cudaHostAllocDefault));
  ZK_CUDA(cudaStreamSynchronize(stream));
  return 0;
}

zk_ctx* zk_ctx::acquire_lane(bool primary_only) {
  std::unique_lock<std::mutex> lk(pool_mu);
  for (;;) {
    if (!busy) {
      busy = true;
      return this;
    }
    if (!primary_only) {
      for (zk_ctx* l : lanes)
        if (!l->busy) {
          l->busy = true;
          return l;
        }
      if ((int)lanes.size() + 1 < max_lanes) {
        zk_ctx* l = new zk_ctx();
        l->device = device;
        l->primary = this;
        l->replicate_entries = replicate_entries;
        l->peer_exchange = peer_exchange;
        l->device_tail = device_tail;
        l->exchange_wait_ms = exchange_wait_ms;
        l->ahead_log = ahead_log;
        if (l->setup() == 0) {
          l->busy = true;
          lanes.push_back(l);
          return l;
        }
        l->teardown();  // no memory for another lane: wait for a free one instead
        delete l;
        max_lanes = (int)lanes.size() + 1;
      }
    }
    pool_cv.wait(lk);
  }
}

void zk_ctx::release_lane(zk_ctx* lane) {
  {
    std::lock_guard<std::mutex> lk(pool_mu);
    lane->busy = false;
  }
  pool_cv.notify_all();
}

uint64_t zk_ctx::total_launches() const {
  uint64_t n = launches.load();
  for (const zk_ctx* l : lanes) n += l->launches.load();
  return n;
}

void zk_ctx::teardown() {
  for (zk_ctx* l : lanes) {
    l->teardown();
    delete l;
  }
  lanes.clear();
  cudaSetDevice(device);
  if (stream) cudaStreamSynchronize(stream);
  if (side_stream) cudaStreamSynchronize(side_stream);
  cudaFree(rs.sink.partials);
  cudaFree(rs.sink.counter);
  cudaFree(rs.sink.msg);
  if (mailbox) cudaFreeHost(mailbox);
  cudaFree(final_out);
  cudaFree(tail_buf);
  cudaFree(tail_out);
  cudaFree(resident_sh);
  cudaFree(work);
  cudaFree(aux);
  cudaFree(cmp);
  if (host_small) cudaFreeHost(host_small);
  for (auto& sp : prof_spans) {
    cudaEventDestroy(sp.e0);
    cudaEventDestroy(sp.e1);
  }
  if (ev_fork) cudaEventDestroy(ev_fork);
  if (ev_join) cudaEventDestroy(ev_join);
  if (side_stream) cudaStreamDestroy(side_stream);
  if (stream) cudaStreamDestroy(stream);
}

static int grow(cudaStream_t stream, void** buf, size_t* have, size_t bytes) {
  if (bytes > *have) {
    ZK_CUDA(cudaStreamSynchronize(stream));
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    const size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
    cudaError_t e = cudaMalloc(buf, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(-2 /*ZK_ERR_OOM*/, "device scratch of %zu bytes: %s", want, cudaGetErrorString(e));
    }
    *have = want;
  }
  return 0;
}

int zk_ctx::reserve_aux(size_t bytes, void** out) {
  int rc = grow(stream, &aux, &aux_bytes, bytes);
  if (rc) return rc;
  *out = aux;
  return 0;
}

int zk_ctx::reserve_cmp(size_t bytes, void** out) {
  int rc = grow(stream, &cmp, &cmp_bytes, bytes);
  if (rc) return rc;
  *out = cmp;
  return 0;
}

int zk_ctx::reserve_work(size_t bytes, void** out) {
  if (bytes > work_bytes) {
    ZK_CUDA(cudaStreamSynchronize(stream));
    if (work) cudaFree(work);
    work = nullptr;
    work_bytes = 0;
    const size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
    cudaError_t e = cudaMalloc(&work, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(-2 /*ZK_ERR_OOM*/, "device scratch of %zu bytes: %s", want, cudaGetErrorString(e));
    }
    work_bytes = want;
  }
  *out = work;
  return 0;
}

void zk_ctx::prof_begin(int kind, double bytes, int n_launches) {
  if (!prof_on) return;
  if (prof_used == prof_spans.size()) {
    ProfSpan sp;
    cudaEventCreate(&sp.e0);
    cudaEventCreate(&sp.e1);
    prof_spans.push_back(sp);
  }
  ProfSpan& sp = prof_spans[prof_used];
  sp.kind = kind;
  prof_launches[kind] += n_launches;
  prof_bytes[kind] += bytes;
  cudaEventRecord(sp.e0, stream);
}

void zk_ctx::prof_end() {
  if (!prof_on) return;
  cudaEventRecord(prof_spans[prof_used].e1, stream);
  prof_used++;
}

int zk_ctx::prof_collect() {
  for (size_t i = 0; i < prof_used; i++) {
    float ms = 0;
    ZK_CUDA(cudaEventSynchronize(prof_spans[i].e1));
    ZK_CUDA(cudaEventElapsedTime(&ms, prof_spans[i].e0, prof_spans[i].e1));
    prof_ms[prof_spans[i].kind] += ms;
  }
  prof_used = 0;
  return 0;
}
