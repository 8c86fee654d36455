#include "ctx.hpp"

using namespace zk;

int zk_ctx::setup() {
  ZK_CUDA(cudaSetDevice(device));
  ZK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  ZK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  rs.max_blocks = sm_count * 8;
  rs.sm_count = sm_count;
  ZK_CUDA(cudaMalloc(&rs.partials, sizeof(Fr) * (size_t)rs.max_blocks * (kMaxPolys + 1)));
  ZK_CUDA(cudaMalloc(&rs.counter, 256));
  ZK_CUDA(cudaMemsetAsync(rs.counter, 0, 256, stream));
  ZK_CUDA(cudaMalloc(&rs.msg, sizeof(Fr) * 16));
  ZK_CUDA(cudaMalloc(&final_out, sizeof(Fr) * 16));
  ZK_CUDA(cudaHostAlloc(&host_small, 4096, cudaHostAllocDefault));
  ZK_CUDA(cudaStreamSynchronize(stream));
  return 0;
}

void zk_ctx::teardown() {
  cudaSetDevice(device);
  if (stream) cudaStreamSynchronize(stream);
  cudaFree(rs.partials);
  cudaFree(rs.counter);
  cudaFree(rs.msg);
  cudaFree(final_out);
  cudaFree(work);
  if (host_small) cudaFreeHost(host_small);
  if (stream) cudaStreamDestroy(stream);
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
