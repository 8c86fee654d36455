// The last rounds of the dense prover in one launch: once the tables are small (at most
// kTailMax entries each) they are kept in shared memory and every remaining round - message,
// Fiat-Shamir step, fold - plus the final product runs without leaving the device, so the per-round
// launch, read-back and host transcript latency disappears.  Only for the built-in transcript: with a
// caller-supplied callback the host has to see every message.
// Rounds: linear_prover.rs:59-72; message :82-140; fold :151-178; final :181-190.
//
// Used where the multi-block kernel of resident.cu does not run to the end by itself: sharded proves, four
// tables, a challenge that is already pending on entry.
#include "internal.hpp"
#include "reduce.cuh"
#include "strobe_dev.cuh"

namespace zk {
namespace {

constexpr int kTailThreads = 256;



template <int L>
struct TailParams {
  const Fr* src[L];
  uint32_t size;    // entries per table on entry
  int fold_first;   // bind `r` on the tables before the first message
  Fr r;
  StrobeState st;
  const Fr* r_dev;            // when set: read r and the transcript state from device memory instead
  const StrobeState* st_dev;
  Fr* out_msgs;     // rounds * (L + 1)
  Fr* out_chal;     // rounds
  Fr* out_final;    // L table values, then their product
  StrobeState* out_st;
};

template <int L>
__global__ void __launch_bounds__(kTailThreads) k_tail(const TailParams<L> p) {
  extern __shared__ uint4 tail_smem[];
  Fr* A = reinterpret_cast<Fr*>(tail_smem);         // L * size
  Fr* B = A + (size_t)L * p.size;                   // L * size / 2
  Fr* red = B + (size_t)L * (p.size / 2 + 1);       // (kTailThreads / 32) * (L + 1)
  Fr* chal = red + (kTailThreads / 32) * (L + 1);   // 1
  __shared__ __align__(16) uint8_t stream[WarpStrobe::round_stream_bytes<L>() + 15];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ __align__(16) uint64_t keccak_scratch[64];
  WarpStrobe ws;                  // live in warp 0 only
  ws.scratch = keccak_scratch;
  if (p.st_dev) {
    ws.a = (warp == 0 && lane < 25) ? p.st_dev->lanes[lane] : 0;
    ws.pos = p.st_dev->pos;
    ws.pos_begin = p.st_dev->pos_begin;
  } else {
    ws.a = (warp == 0 && lane < 25) ? p.st.lanes[lane] : 0;
    ws.pos = p.st.pos;
    ws.pos_begin = p.st.pos_begin;
  }
  if (tid == 0) WarpStrobe::init_round_stream<L>(stream);

  for (uint32_t i = tid; i < p.size; i += kTailThreads)
#pragma unroll
    for (int t = 0; t < L; t++) A[(size_t)t * p.size + i] = p.src[t][i];
  if (tid == 0) chal[0] = p.r_dev ? *p.r_dev : p.r;
  __syncthreads();

  Fr* cur = A;
  Fr* nxt = B;
  uint32_t cur_size = p.size, cur_stride = p.size, nxt_stride = p.size / 2 + 1;
  bool fold_now = p.fold_first != 0;
  uint32_t round = 0;
  while (true) {
    if (fold_now) {
      const Fr r = chal[0];
      const uint32_t half = cur_size >> 1;
      for (uint32_t y = tid; y < half; y += kTailThreads)
#pragma unroll
        for (int t = 0; t < L; t++) {
          const Fr a0 = cur[(size_t)t * cur_stride + 2 * y], a1 = cur[(size_t)t * cur_stride + 2 * y + 1];
          nxt[(size_t)t * nxt_stride + y] = add(a0, mul(r, sub(a1, a0)));
        }
      __syncthreads();
      Fr* tmp = cur; cur = nxt; nxt = tmp;
      const uint32_t ts = cur_stride; cur_stride = nxt_stride; nxt_stride = ts;
      cur_size = half;
    }
    if (cur_size <= 1) break;
    // ---- message of this round
    Fr s[L + 1];
#pragma unroll
    for (int c = 0; c <= L; c++) s[c] = Fr::zero();
    const uint32_t pairs = cur_size >> 1;
    for (uint32_t y = tid; y < pairs; y += kTailThreads) {
      Fr v[L], d[L];
#pragma unroll
      for (int t = 0; t < L; t++) {
        v[t] = cur[(size_t)t * cur_stride + 2 * y];
        d[t] = sub(cur[(size_t)t * cur_stride + 2 * y + 1], v[t]);
      }
#pragma unroll
      for (int c = 0; c <= L; c++) {
        Fr prod = v[0];
#pragma unroll
        for (int t = 1; t < L; t++) prod = mul(prod, v[t]);
        s[c] = add(s[c], prod);
        if (c < L) {
#pragma unroll
          for (int t = 0; t < L; t++) v[t] = add(v[t], d[t]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c <= L; c++) {
      const Fr t = warp_sum(s[c]);
      if (lane == 0) red[warp * (L + 1) + c] = t;
    }
    __syncthreads();
    if (warp == 0) {
      // Fiat-Shamir step by the whole first warp (transcript.rs:27-42 over STROBE / Keccak-f)
      if (lane <= L) {  // one lane per evaluation: total, canonical form, bytes
        Fr t = red[lane];
        for (int w = 1; w < kTailThreads / 32; w++) t = add(t, red[w * (L + 1) + lane]);
        p.out_msgs[(size_t)round * (L + 1) + lane] = t;
        const Fr canon = from_mont(t);
        uint8_t* dst = WarpStrobe::round_stream_data(stream, lane);
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
          for (int k = 0; k < 4; k++) dst[4 * i + k] = (uint8_t)(canon.v[i] >> (8 * k));
      }
      __syncwarp();
      Fr raw;
      ws.fs_round<L>(stream, lane, raw.v);
      if (lane == 0) {
        const Fr ch = to_mont(raw);
        p.out_chal[round] = ch;
        chal[0] = ch;
      }
    }
    __syncthreads();
    fold_now = true;
    round++;
  }
  if (tid == 0) {
    Fr prod = Fr::one();
    for (int t = 0; t < L; t++) {
      const Fr a = cur[(size_t)t * cur_stride];
      p.out_final[t] = a;
      prod = mul(prod, a);
    }
    p.out_final[L] = prod;
    p.out_st->pos = ws.pos;
    p.out_st->pos_begin = ws.pos_begin;
    p.out_st->cur_flags = 1u | 2u | 4u;  // the last operation was the PRF of a challenge (or nothing ran)
    p.out_st->pad = 0;
  }
  if (warp == 0 && lane < 25) p.out_st->lanes[lane] = ws.a;
}

template <int L>
int launch_tail_t(const Fr* const* src, uint32_t size, bool fold_first, const Fr& r, const StrobeState& st, Fr* out_msgs,
                  Fr* out_chal, Fr* out_final, StrobeState* out_st, cudaStream_t stream, const Fr* r_dev,
                  const StrobeState* st_dev) {
  TailParams<L> q;
  q.r_dev = r_dev;
  q.st_dev = st_dev;
  for (int i = 0; i < L; i++) q.src[i] = src[i];
  q.size = size;
  q.fold_first = fold_first ? 1 : 0;
  q.r = r;
  q.st = st;
  q.out_msgs = out_msgs;
  q.out_chal = out_chal;
  q.out_final = out_final;
  q.out_st = out_st;
  const size_t smem1 = ((size_t)L * size + (size_t)L * (size / 2 + 1) + (kTailThreads / 32) * (L + 1) + 2) * sizeof(Fr);
  if (cudaFuncSetAttribute(k_tail<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -3;
  k_tail<L><<<1, kTailThreads, smem1, stream>>>(q);
  return 0;
}

}  // namespace

int launch_tail(int num_poly, const Fr* const* src, uint32_t size, bool fold_first, const Fr& r, const StrobeState& st,
                Fr* out_msgs, Fr* out_chal, Fr* out_final, StrobeState* out_st, cudaStream_t stream, const Fr* r_dev,
                const StrobeState* st_dev) {
  switch (num_poly) {
    case 1: return launch_tail_t<1>(src, size, fold_first, r, st, out_msgs, out_chal, out_final, out_st, stream, r_dev, st_dev);
    case 2: return launch_tail_t<2>(src, size, fold_first, r, st, out_msgs, out_chal, out_final, out_st, stream, r_dev, st_dev);
    case 3: return launch_tail_t<3>(src, size, fold_first, r, st, out_msgs, out_chal, out_final, out_st, stream, r_dev, st_dev);
    case 4: return launch_tail_t<4>(src, size, fold_first, r, st, out_msgs, out_chal, out_final, out_st, stream, r_dev, st_dev);
    default: return -1;
  }
}

}  // namespace zk
