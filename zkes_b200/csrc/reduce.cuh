// Device helpers shared by the kernels: element <-> 128-bit chunk packing and the
// warp / block / grid reduction of field elements.
#pragma once
#include "ff.cuh"
#include "internal.hpp"
#include <cuda_runtime.h>

namespace zk {

__device__ __forceinline__ Fr fr_from_chunks(const uint4& lo, const uint4& hi) {
  Fr x;
  x.v[0] = lo.x; x.v[1] = lo.y; x.v[2] = lo.z; x.v[3] = lo.w;
  x.v[4] = hi.x; x.v[5] = hi.y; x.v[6] = hi.z; x.v[7] = hi.w;
  return x;
}
__device__ __forceinline__ void fr_to_chunks(const Fr& x, uint4& lo, uint4& hi) {
  lo = make_uint4(x.v[0], x.v[1], x.v[2], x.v[3]);
  hi = make_uint4(x.v[4], x.v[5], x.v[6], x.v[7]);
}

__device__ __forceinline__ void st_fr_sys(Fr* p, const Fr& x) {
  volatile uint32_t* q = reinterpret_cast<volatile uint32_t*>(p);
#pragma unroll
  for (int i = 0; i < 8; i++) q[i] = x.v[i];
}

__device__ __forceinline__ Fr shfl_down_fr(const Fr& x, int delta) {
  Fr r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = __shfl_down_sync(0xffffffffu, x.v[i], delta);
  return r;
}

__device__ __forceinline__ Fr warp_sum(Fr s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s = add(s, shfl_down_fr(s, off));
  return s;  // lane 0 holds the total
}

__device__ __forceinline__ Fr ld_cg_fr(const Fr* p) {
  const uint4 lo = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint4 hi = __ldcg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}

// Sum NV per-thread values over the grid; the last block to arrive writes out[0..NV).
// partials holds gridDim.x * NV elements; *counter must be zero on entry and is reset.
template <int NV, int kWarps>
__device__ __forceinline__ void grid_sum(Fr (&s)[NV], const MsgSink& sink) {
  Fr* partials = sink.partials;
  unsigned int* counter = sink.counter;
  Fr* out = sink.msg;
  __shared__ Fr sh[kWarps][NV];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int c = 0; c < NV; c++) {
    Fr t = warp_sum(s[c]);
    if (lane == 0) sh[warp][c] = t;
  }
  __syncthreads();
  if (threadIdx.x < NV) {
    Fr t = sh[0][threadIdx.x];
    for (int w = 1; w < kWarps; w++) t = add(t, sh[w][threadIdx.x]);
    partials[(size_t)blockIdx.x * NV + threadIdx.x] = t;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
#pragma unroll
  for (int c = 0; c < NV; c++) {
    Fr t = Fr::zero();
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x) t = add(t, ld_cg_fr(partials + (size_t)b * NV + c));
    t = warp_sum(t);
    if (lane == 0) sh[warp][c] = t;
  }
  __syncthreads();
  if (threadIdx.x < NV) {
    Fr t = sh[0][threadIdx.x];
    for (int w = 1; w < kWarps; w++) t = add(t, sh[w][threadIdx.x]);
    out[threadIdx.x] = t;
    if (sink.pub_flag) st_fr_sys(sink.pub_msg + threadIdx.x, t);
  }
  if (threadIdx.x == 0) *counter = 0;
  if (sink.pub_flag) {  // publish to the polling host: data, system-wide fence, then the sequence word
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag) = sink.seq;
  }
}

// grid_sum for one rank of a sharded instance: the last block to arrive also exchanges the totals with the other
// ranks' kernels through the peer boxes (every rank's kernel does the same at its end), adds the shares in rank
// order and publishes the complete message, with the outcome of the wait in the word beside the sequence word:
// the exchange needs no launch of its own.  sink.pub_flag must be set.
template <int NV, int kWarps>
__device__ __forceinline__ void grid_sum_exchange(Fr (&s)[NV], const MsgSink& sink, const PeerExchange& px, unsigned int xseq) {
  Fr* partials = sink.partials;
  unsigned int* counter = sink.counter;
  __shared__ Fr sh[kWarps][NV];
  __shared__ Fr tot[NV];
  __shared__ uint32_t stage[kPeerRanks * NV * 8];
  __shared__ int ok_shared;
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int c = 0; c < NV; c++) {
    Fr t = warp_sum(s[c]);
    if (lane == 0) sh[warp][c] = t;
  }
  __syncthreads();
  if (threadIdx.x < NV) {
    Fr t = sh[0][threadIdx.x];
    for (int w = 1; w < kWarps; w++) t = add(t, sh[w][threadIdx.x]);
    partials[(size_t)blockIdx.x * NV + threadIdx.x] = t;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(counter, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
#pragma unroll
  for (int c = 0; c < NV; c++) {
    Fr t = Fr::zero();
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x) t = add(t, ld_cg_fr(partials + (size_t)b * NV + c));
    t = warp_sum(t);
    if (lane == 0) sh[warp][c] = t;
  }
  __syncthreads();
  if (threadIdx.x < NV) {
    Fr t = sh[0][threadIdx.x];
    for (int w = 1; w < kWarps; w++) t = add(t, sh[w][threadIdx.x]);
    tot[threadIdx.x] = t;
  }
  if (threadIdx.x == 0) *counter = 0;
  __syncthreads();
  const bool ok = peer_exchange_sum(px, xseq, tot, NV, stage, &ok_shared, threadIdx.x, blockDim.x);
  if (threadIdx.x < NV && ok) {
    sink.msg[threadIdx.x] = tot[threadIdx.x];
    st_fr_sys(sink.pub_msg + threadIdx.x, tot[threadIdx.x]);
  }
  if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag + 1) = ok ? 0u : 1u;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(sink.pub_flag) = sink.seq;
}

}  // namespace zk
