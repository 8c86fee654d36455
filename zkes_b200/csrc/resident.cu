// Several rounds of the dense prover in one cooperative launch.
//
// With the built-in transcript nothing of a round has to leave the device: every block folds and
// sums its share of the tables, the last block to arrive adds the partial messages, runs the
// Fiat-Shamir step (one warp, transcript.rs:27-42 over STROBE / Keccak-f), and publishes the
// challenge's multiplier table; the other blocks wait for it and start the next round.  That
// replaces a launch, a read-back and a host transcript step per round by one device-side
// hand-over.  The launch is cooperative so that all blocks are resident together; every wait is
// bounded and reports through ResidentShared::error instead of spinning on.
// Rounds: linear_prover.rs:59-72; message :82-140; fold :151-178.
#include <cstring>
#include "internal.hpp"
#include "round_pass.cuh"
#include "strobe_dev.cuh"

namespace zk {
namespace {

constexpr int kThreads = kRoundThreads;
constexpr int kWarps = kRoundWarps;

template <int L>
struct ResidentParams {
  const Fr* src[L];
  Fr* ping[L];
  Fr* pong[L];
  uint64_t size;        // entries per table on entry (a power of two, at least 4)
  uint32_t rounds;      // messages to produce; the last challenge is left unbound
  uint32_t spin_limit;  // polls before a wait gives up
  StrobeState st;       // transcript state on entry
  Fr* partials;         // gridDim.x * (L + 1)
  ResidentShared* sh;   // zeroed arrive / seq / error on entry
  Fr* out_msgs;         // rounds * (L + 1)
  Fr* out_chal;         // rounds
  Fr pow2[8];           // 2^(32 j + 64) mod r as plain integers: rows of a multiplier table
  PeerExchange px;      // px.world > 1: sharded instance, messages are summed over the ranks
};

template <int L>
__global__ void __launch_bounds__(kThreads, (L <= 1 ? 3 : 2)) k_resident(const ResidentParams<L> p) {
  __shared__ uint4 stage[kWarps][WarpTile<8>::kChunks];
  __shared__ FixedMul<FrParams> r_tab;
  __shared__ Fr red[kWarps][L + 1];
  __shared__ Fr msg[L + 1];
  __shared__ __align__(16) uint8_t stream[WarpStrobe::round_stream_bytes<L>() + 15];
  __shared__ int flag, ok_flag, px_ok;
  __shared__ uint32_t px_stage[kPeerRanks * (L + 1) * 8];
  __shared__ __align__(16) uint64_t keccak_scratch[64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int NV = L + 1;
  if (threadIdx.x == 0) WarpStrobe::init_round_stream<L>(stream);

  const Fr* cur[L];
#pragma unroll
  for (int i = 0; i < L; i++) cur[i] = p.src[i];
  uint64_t cur_size = p.size;
  const uint64_t warp_global = (uint64_t)blockIdx.x * kWarps + warp, warp_stride = (uint64_t)gridDim.x * kWarps;

  for (uint32_t round = 0; round < p.rounds; round++) {
    Fr s[NV];
    if (round == 0) {
      round_pass<L, false, false>(cur, cur, r_tab, cur_size >> 1, warp_global, warp_stride, stage[warp], lane, s);
    } else {
      Fr* dst[L];
#pragma unroll
      for (int i = 0; i < L; i++) dst[i] = (round & 1) ? p.ping[i] : p.pong[i];
      round_pass<L, true, true>(cur, dst, r_tab, cur_size >> 2, warp_global, warp_stride, stage[warp], lane, s);
#pragma unroll
      for (int i = 0; i < L; i++) cur[i] = dst[i];
      cur_size >>= 1;
    }
    // block total -> global; the last block to arrive owns the rest of the round.  Only blocks that
    // had tiles this round hold a non-zero share: the others skip the store and are not read.
    const uint64_t tiles = ((cur_size >> 1) + 31) >> 5;  // cur_size: entries of the table the message is over
    const unsigned int active = (unsigned int)((tiles + kWarps - 1) / kWarps < gridDim.x ? (tiles + kWarps - 1) / kWarps : gridDim.x);
    if (blockIdx.x < active) {
#pragma unroll
      for (int c = 0; c < NV; c++) {
        const Fr t = warp_sum(s[c]);
        if (lane == 0) red[warp][c] = t;
      }
      __syncthreads();
      if (threadIdx.x < NV) {
        Fr t = red[0][threadIdx.x];
        for (int w = 1; w < kWarps; w++) t = add(t, red[w][threadIdx.x]);
        p.partials[(size_t)blockIdx.x * NV + threadIdx.x] = t;
      }
      __threadfence();  // this block's folded entries and its share, before the ticket
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int ticket = atomicAdd(&p.sh->arrive, 1u);
      flag = ticket == (round + 1) * gridDim.x - 1;
    }
    __syncthreads();
    if (flag) {
      __threadfence();
      // NV * active values over the block: all of a thread's loads are issued before its additions
      Fr t[NV];
#pragma unroll
      for (int c = 0; c < NV; c++) t[c] = Fr::zero();
      for (unsigned int b0 = 0; b0 < active; b0 += 2 * kThreads) {
        const unsigned int b1 = b0 + threadIdx.x, b2 = b1 + kThreads;
        Fr u[NV], v[NV];
#pragma unroll
        for (int c = 0; c < NV; c++) {
          u[c] = b1 < active ? ld_cg_fr(p.partials + (size_t)b1 * NV + c) : Fr::zero();
          v[c] = b2 < active ? ld_cg_fr(p.partials + (size_t)b2 * NV + c) : Fr::zero();
        }
#pragma unroll
        for (int c = 0; c < NV; c++) t[c] = add(t[c], add(u[c], v[c]));
      }
#pragma unroll
      for (int c = 0; c < NV; c++) {
        const Fr w = warp_sum(t[c]);
        if (lane == 0) red[warp][c] = w;
      }
      __syncthreads();
      if (threadIdx.x < NV) {
        Fr w = red[0][threadIdx.x];
        for (int k = 1; k < kWarps; k++) w = add(w, red[k][threadIdx.x]);
        msg[threadIdx.x] = w;
      }
      __syncthreads();
      if (p.px.world > 1) {
        // Sharded instance: msg holds this rank's share.  Store it into every rank's box, wait (bounded)
        // for the other ranks' shares in this rank's own box and add them in rank order, so every rank
        // absorbs the same message and derives the same challenge.
        const unsigned int xseq = p.px.xseq_base + round + 1;
        if (!peer_exchange_sum(p.px, xseq, msg, NV, px_stage, &px_ok, threadIdx.x, kThreads)) {
          if (threadIdx.x == 0) atomicExch(&p.sh->error, 2u);  // a rank is missing: stops every block of this launch
          return;
        }
      }
      if (warp == 0) {
        WarpStrobe ws;
        ws.scratch = keccak_scratch;
        if (round == 0) {
          ws.a = lane < 25 ? p.st.lanes[lane] : 0;
          ws.pos = p.st.pos;
          ws.pos_begin = p.st.pos_begin;
        } else {
          ws.a = lane < 25 ? __ldcg(reinterpret_cast<const unsigned long long*>(&p.sh->st.lanes[lane])) : 0;
          ws.pos = __ldcg(&p.sh->st.pos);
          ws.pos_begin = __ldcg(&p.sh->st.pos_begin);
        }
        if (lane <= L) {
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
        if (lane < 8) {  // eight lanes build the eight rows of the challenge's multiplier table
          const Fr ch = to_mont(raw);
          const Fr row = mul(ch, p.pow2[lane]);
#pragma unroll
          for (int k = 0; k < 8; k++) p.sh->table.c[lane][k] = row.v[k];
          if (lane == 0) {
            p.out_chal[round] = ch;
            p.sh->challenge = ch;
            p.sh->st.pos = ws.pos;
            p.sh->st.pos_begin = ws.pos_begin;
            p.sh->st.cur_flags = 1u | 2u | 4u;
            p.sh->st.pad = 0;
          }
        }
        if (lane < 25) p.sh->st.lanes[lane] = ws.a;
        __threadfence();
        __syncwarp();
        if (lane == 0) *reinterpret_cast<volatile unsigned int*>(&p.sh->seq) = round + 1;
      }
    }
    if (round + 1 == p.rounds) break;  // the last challenge is consumed by whoever runs next
    // wait for this round's challenge
    if (threadIdx.x == 0) {
      const volatile unsigned int* seq = reinterpret_cast<const volatile unsigned int*>(&p.sh->seq);
      const volatile unsigned int* err = reinterpret_cast<const volatile unsigned int*>(&p.sh->error);
      uint32_t polls = 0;
      int ok = 1;
      while (*seq < round + 1) {
        if (*err != 0) {  // another block gave up and said why: leave its code in place
          ok = 0;
          break;
        }
        if (++polls > p.spin_limit) {
          atomicCAS(&p.sh->error, 0u, 1u);
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
      __threadfence();
      ok_flag = ok;
    }
    __syncthreads();
    if (!ok_flag) return;
    if (threadIdx.x < 64) (&r_tab.c[0][0])[threadIdx.x] = __ldcg(&p.sh->table.c[0][0] + threadIdx.x);
    __syncthreads();
  }
}

template <int L>
int launch_resident_t(const Fr* const* src, Fr* const* ping, Fr* const* pong, uint64_t size, uint32_t rounds,
                      const StrobeState& st, Fr* partials, int max_blocks, int sm_count, ResidentShared* sh, Fr* out_msgs,
                      Fr* out_chal, cudaStream_t stream, const PeerExchange* px) {
  ResidentParams<L> p;
  if (px) {
    p.px = *px;
  } else {
    memset(&p.px, 0, sizeof p.px);
    p.px.world = 1;
  }
  for (int i = 0; i < L; i++) {
    p.src[i] = src[i];
    p.ping[i] = ping[i];
    p.pong[i] = pong[i];
  }
  p.size = size;
  p.rounds = rounds;
  // with the 64 ns pause between polls: seconds; sharded, the blocks also sit out the wait of the block
  // that exchanges with the other ranks, which tolerates ranks that start seconds apart
  p.spin_limit = px ? 3u * px->spin_limit : (8u << 20);
  p.st = st;
  p.partials = partials;
  p.sh = sh;
  p.out_msgs = out_msgs;
  p.out_chal = out_chal;
  Fr cur = Fr::zero();
  cur.v[2] = 1;  // 2^64
  Fr step = Fr::zero();
  step.v[1] = 1;
  step = to_mont(step);  // (2^32) R: a Montgomery product with it multiplies a plain integer by 2^32
  for (int j = 0; j < 8; j++) {
    p.pow2[j] = cur;
    cur = mul(cur, step);
  }
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_resident<L>, kThreads, 0) != cudaSuccess || occ < 1) return -2;
  uint64_t grid = ((size >> 1) + 31) / 32;  // tiles of the first round
  grid = (grid + kWarps - 1) / kWarps;
  const uint64_t cap = (uint64_t)sm_count * occ < (uint64_t)max_blocks ? (uint64_t)sm_count * occ : (uint64_t)max_blocks;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  void* args[] = {&p};
  if (cudaMemsetAsync(sh, 0, 16, stream) != cudaSuccess) return -3;
  if (cudaLaunchCooperativeKernel((const void*)k_resident<L>, dim3((unsigned)grid), dim3(kThreads), args, 0, stream) !=
      cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}

}  // namespace

// Runs `rounds` rounds on tables of `size` entries.  Afterwards the tables that the last fold
// wrote are ((rounds - 1) & 1 ? ping : pong) for rounds >= 2 (src for rounds == 1), the last
// challenge is in sh->challenge and the transcript state in sh->st.  Non-zero: the cooperative
// launch was not possible and nothing ran.
int launch_resident(int num_poly, const Fr* const* src, Fr* const* ping, Fr* const* pong, uint64_t size, uint32_t rounds,
                    const StrobeState& st, Fr* partials, int max_blocks, int sm_count, ResidentShared* sh, Fr* out_msgs,
                    Fr* out_chal, cudaStream_t stream, const PeerExchange* px) {
  switch (num_poly) {
    case 1: return launch_resident_t<1>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px);
    case 2: return launch_resident_t<2>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px);
    case 3: return launch_resident_t<3>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px);
    case 4: return launch_resident_t<4>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px);
    default: return -1;
  }
}

}  // namespace zk
