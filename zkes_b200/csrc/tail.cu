// The last rounds of the dense prover in one launch: once the tables are small (at most
// kTailMax entries each) they are kept in shared memory and every remaining round - message,
// Fiat-Shamir step, fold - plus the final product runs without leaving the device, so the per-round
// launch, read-back and host transcript latency disappears.  Only for the built-in transcript: with a
// caller-supplied callback the host has to see every message.
// Rounds: linear_prover.rs:59-72; message :82-140; fold :151-178; final :181-190.
//
// The transcript step of a round (two Keccak permutations by one warp, about 6 us) is longer than the table
// work of a round at these sizes, and the rounds depend on one another through the challenge.  k_tail takes
// the table work off that chain with a cluster of two blocks on two SMs: block 0 hashes, block 1 holds the
// tables.  While block 0 hashes the message of round t, block 1 prepares round t + 1 without knowing the
// challenge r_t: folding by r_t is linear in r_t, so the next message is a polynomial of degree L in r_t,
//     s_{t+1}(c) = G(c, r_t),   G(c, rho) = sum_y prod_i bilinear(T_i[4y .. 4y+3]; rho, c),
// the round polynomial of two variables at once.  Block 1 tabulates G on the grid {0..L} x {0..L} and stores
// it into block 0's shared memory; when r_t is out, block 0 interpolates s_{t+1} (a few products), goes
// straight on to hash it and hands r_t to block 1, which folds the tables by it and tabulates the grid of
// the round after.  One cluster barrier per round separates the phases; every value is an exact field
// element, so the messages are the reference's, bit for bit.  (On one SM the same scheme was slower than
// the plain loop: the worker warps and the hashing warp slow one another down.)  k_tail_single is the plain
// loop in one block, used when a cluster launch is not available.
#include <cooperative_groups.h>

#include "internal.hpp"
#include "reduce.cuh"
#include "strobe_dev.cuh"

namespace cg = cooperative_groups;

namespace zk {
namespace {

constexpr int kTailThreads = 256;



template <int L>
struct TailParamsSingle {
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
__global__ void __launch_bounds__(kTailThreads) k_tail_single(const TailParamsSingle<L> p) {
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
  Fr node[L + 1];   // the integers 0 .. L (Montgomery form): interpolation nodes
  Fr dinv[L + 1];   // 1 / prod_{k != j} (j - k)
};

template <int L>
__global__ void __launch_bounds__(kTailThreads) k_tail(const TailParams<L> p) {
  constexpr int NV = L + 1, NG = NV * NV;
  cg::cluster_group cluster = cg::this_cluster();
  const bool hasher = cluster.block_rank() == 0;   // block 0: transcript chain; block 1: tables
  extern __shared__ uint4 tail_smem[];
  // the same layout in both blocks; block 1 uses the tables, block 0 the grid and the message
  Fr* A = reinterpret_cast<Fr*>(tail_smem);         // L * size
  Fr* B = A + (size_t)L * p.size;                   // L * (size / 2 + 1)
  Fr* red = B + (size_t)L * (p.size / 2 + 1);       // 8 * NG: per-warp partial sums
  Fr* gsum = red + 8 * NG;                          // 2 * NG: grid of the next message, double-buffered (block 0's copy is live)
  Fr* msg = gsum + 2 * NG;                          // NV: the message being hashed (block 0's copy is live)
  Fr* chal = msg + NV;                              // 2: challenges, double-buffered (both copies live)
  Fr* lag = chal + 2;                               // NG: interpolation terms (block 0)
  Fr* gsum_h = cluster.map_shared_rank(gsum, 0);    // block 0's grid and message, as block 1 addresses them
  Fr* msg_h = cluster.map_shared_rank(msg, 0);
  Fr* chal_w = cluster.map_shared_rank(chal, 1);    // block 1's challenges, as block 0 addresses them
  __shared__ __align__(16) uint8_t stream[WarpStrobe::round_stream_bytes<L>() + 15];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ __align__(16) uint64_t keccak_scratch[64];
  WarpStrobe ws;                  // live in warp 0 of block 0 only
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

  Fr* cur = A;
  Fr* nxt = B;
  uint32_t cur_size = p.size, cur_stride = p.size, nxt_stride = p.size / 2 + 1;
  if (!hasher) {
    for (uint32_t i = tid; i < p.size; i += kTailThreads)
#pragma unroll
      for (int t = 0; t < L; t++) A[(size_t)t * p.size + i] = p.src[t][i];
    if (tid == 0) chal[1] = p.r_dev ? *p.r_dev : p.r;
    __syncthreads();
  }
  if (p.fold_first) {  // a challenge the caller (or the kernel before this one) has drawn already
    const uint32_t half = cur_size >> 1;
    if (!hasher) {
      const Fr r = chal[1];
      for (uint32_t y = tid; y < half; y += kTailThreads)
#pragma unroll
        for (int t = 0; t < L; t++) {
          const Fr a0 = cur[(size_t)t * cur_stride + 2 * y], a1 = cur[(size_t)t * cur_stride + 2 * y + 1];
          nxt[(size_t)t * nxt_stride + y] = add(a0, mul(r, sub(a1, a0)));
        }
      __syncthreads();
    }
    Fr* tmp = cur; cur = nxt; nxt = tmp;
    const uint32_t ts = cur_stride; cur_stride = nxt_stride; nxt_stride = ts;
    cur_size = half;
  }
  uint32_t round = 0;
  if (cur_size > 1) {
    if (!hasher) {
      // ---- the first message, straight from the table, into block 0's shared memory
      Fr s[NV];
#pragma unroll
      for (int c = 0; c < NV; c++) s[c] = Fr::zero();
      const uint32_t pairs = cur_size >> 1;
      for (uint32_t y = tid; y < pairs; y += kTailThreads) {
        Fr v[L], d[L];
#pragma unroll
        for (int t = 0; t < L; t++) {
          v[t] = cur[(size_t)t * cur_stride + 2 * y];
          d[t] = sub(cur[(size_t)t * cur_stride + 2 * y + 1], v[t]);
        }
#pragma unroll
        for (int c = 0; c < NV; c++) {
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
      for (int c = 0; c < NV; c++) {
        const Fr t = warp_sum(s[c]);
        if (lane == 0) red[warp * NV + c] = t;
      }
      __syncthreads();
      if (tid < NV) {
        Fr t = red[tid];
        for (int w = 1; w < kTailThreads / 32; w++) t = add(t, red[w * NV + tid]);
        msg_h[tid] = t;
      }
    }
    cluster.sync();

    // ---- phases: block 0 hashes the message of round `round`; block 1 binds the previous challenge and
    // tabulates the grid of the next message.  cur holds the tables the message of round `round` is over,
    // except that in phases after the first block 1 still has to bind chal[(round - 1) & 1] on them.
    bool fold_pending = false;
    while (true) {
      const uint32_t size_now = fold_pending ? cur_size >> 1 : cur_size;  // entries of the tables of this round's message
      if (hasher) {
        if (warp == 0) {
          if (round > 0) {
            // s_round(c) = sum_j lambda_j(r) G(c, j), r = the challenge of the round before
            const Fr r = chal[(round - 1) & 1];
            if (lane < NG) {
              const int j = lane % NV;
              Fr lam = p.dinv[j];
#pragma unroll
              for (int k = 0; k < NV; k++)
                if (k != j) lam = mul(lam, sub(r, p.node[k]));
              lag[lane] = mul(lam, gsum[(round & 1) * NG + lane]);
            }
            __syncwarp();
            if (lane < NV) {
              Fr t = lag[lane * NV];
#pragma unroll
              for (int j = 1; j < NV; j++) t = add(t, lag[lane * NV + j]);
              msg[lane] = t;
            }
            __syncwarp();
          }
          // Fiat-Shamir step by the whole first warp (transcript.rs:27-42 over STROBE / Keccak-f)
          if (lane <= L) {  // one lane per evaluation: canonical form, bytes
            const Fr t = msg[lane];
            p.out_msgs[(size_t)round * NV + lane] = t;
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
            chal[round & 1] = ch;      // for this block's interpolation of the next message
            chal_w[round & 1] = ch;    // for block 1's fold
          }
        }
      } else {
        if (fold_pending) {
          const Fr r = chal[(round - 1) & 1];
          const uint32_t half = cur_size >> 1;
          for (uint32_t y = tid; y < half; y += kTailThreads)
#pragma unroll
            for (int t = 0; t < L; t++) {
              const Fr a0 = cur[(size_t)t * cur_stride + 2 * y], a1 = cur[(size_t)t * cur_stride + 2 * y + 1];
              nxt[(size_t)t * nxt_stride + y] = add(a0, mul(r, sub(a1, a0)));
            }
          __syncthreads();
        }
        // the tables of this round's message, and the grid of the next one over their quads
        const Fr* tab = fold_pending ? nxt : cur;
        const uint32_t stride = fold_pending ? nxt_stride : cur_stride;
        if (size_now >= 4) {
          Fr g[NG];
#pragma unroll
          for (int v = 0; v < NG; v++) g[v] = Fr::zero();
          const uint32_t quads = size_now >> 2;
          for (uint32_t q = tid; q < quads; q += kTailThreads) {
            Fr e0[L], e1[L], d0[L], d1[L];
#pragma unroll
            for (int t = 0; t < L; t++) {
              const Fr* v = tab + (size_t)t * stride + 4 * q;
              e0[t] = v[0];
              d0[t] = sub(v[1], v[0]);
              e1[t] = v[2];
              d1[t] = sub(v[3], v[2]);
            }
#pragma unroll
            for (int rho = 0; rho < NV; rho++) {
              Fr x[L], dx[L];
#pragma unroll
              for (int t = 0; t < L; t++) {
                x[t] = e0[t];
                dx[t] = sub(e1[t], e0[t]);
              }
#pragma unroll
              for (int c = 0; c < NV; c++) {
                Fr prod = x[0];
#pragma unroll
                for (int t = 1; t < L; t++) prod = mul(prod, x[t]);
                g[c * NV + rho] = add(g[c * NV + rho], prod);
                if (c < L) {
#pragma unroll
                  for (int t = 0; t < L; t++) x[t] = add(x[t], dx[t]);
                }
              }
              if (rho < L) {
#pragma unroll
                for (int t = 0; t < L; t++) {
                  e0[t] = add(e0[t], d0[t]);
                  e1[t] = add(e1[t], d1[t]);
                }
              }
            }
          }
          const uint32_t live_warps = (quads + 31) / 32 < (uint32_t)(kTailThreads / 32) ? (quads + 31) / 32 : kTailThreads / 32;
          if ((uint32_t)warp < live_warps) {
#pragma unroll
            for (int v = 0; v < NG; v++) {
              const Fr t = warp_sum(g[v]);
              if (lane == 0) red[warp * NG + v] = t;
            }
          }
          __syncthreads();
          if (tid < NG) {
            Fr t = red[tid];
            for (uint32_t k = 1; k < live_warps; k++) t = add(t, red[k * NG + tid]);
            gsum_h[((round + 1) & 1) * NG + tid] = t;
          }
        }
      }
      cluster.sync();
      if (fold_pending) {
        Fr* tmp = cur; cur = nxt; nxt = tmp;
        const uint32_t ts = cur_stride; cur_stride = nxt_stride; nxt_stride = ts;
        cur_size >>= 1;
      }
      fold_pending = true;
      round++;
      if (cur_size == 2) break;  // the challenge just drawn is the last: bound below
    }
  }
  if (!hasher && tid == 0) {
    Fr prod = Fr::one();
    for (int t = 0; t < L; t++) {
      Fr a = cur[(size_t)t * cur_stride];
      if (cur_size == 2) {  // bind the last challenge
        const Fr a1 = cur[(size_t)t * cur_stride + 1];
        a = add(a, mul(chal[(round - 1) & 1], sub(a1, a)));
      }
      p.out_final[t] = a;
      prod = mul(prod, a);
    }
    p.out_final[L] = prod;
  }
  if (hasher && tid == 0) {
    p.out_st->pos = ws.pos;
    p.out_st->pos_begin = ws.pos_begin;
    p.out_st->cur_flags = 1u | 2u | 4u;  // the last operation was the PRF of a challenge (or nothing ran)
    p.out_st->pad = 0;
  }
  if (hasher && warp == 0 && lane < 25) p.out_st->lanes[lane] = ws.a;
}

template <int L>
int launch_tail_t(const Fr* const* src, uint32_t size, bool fold_first, const Fr& r, const StrobeState& st, Fr* out_msgs,
                  Fr* out_chal, Fr* out_final, StrobeState* out_st, cudaStream_t stream, const Fr* r_dev,
                  const StrobeState* st_dev) {
  TailParams<L> p;
  p.r_dev = r_dev;
  p.st_dev = st_dev;
  for (int i = 0; i < L; i++) p.src[i] = src[i];
  p.size = size;
  p.fold_first = fold_first ? 1 : 0;
  p.r = r;
  p.st = st;
  p.out_msgs = out_msgs;
  p.out_chal = out_chal;
  p.out_final = out_final;
  p.out_st = out_st;
  for (int j = 0; j <= L; j++) {
    p.node[j] = from_u32<FrParams>((uint32_t)j);
    Fr den = Fr::one();
    for (int k = 0; k <= L; k++) {
      if (k == j) continue;
      const Fr d = j > k ? from_u32<FrParams>((uint32_t)(j - k)) : neg(from_u32<FrParams>((uint32_t)(k - j)));
      den = mul(den, d);
    }
    p.dinv[j] = inverse(den);
  }
  constexpr int NV = L + 1, NG = NV * NV;
  const size_t smem = ((size_t)L * size + (size_t)L * (size / 2 + 1) + 8 * NG + 2 * NG + NV + 2 + NG + 2) * sizeof(Fr);
  // the opt-in is per device, and a process may hold contexts on several: set it on every launch
  if (cudaFuncSetAttribute(k_tail<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(kTailThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, k_tail<L>, p) == cudaSuccess) return 0;
  }
  cudaGetLastError();
  // no cluster launch on this device: the plain loop in one block
  TailParamsSingle<L> q;
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
  if (cudaFuncSetAttribute(k_tail_single<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -3;
  k_tail_single<L><<<1, kTailThreads, smem1, stream>>>(q);
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
