// Dense sumcheck round kernels over BN254 Fr.
//
// One launch per round.  k_round<L, FOLD> binds the previous round's challenge (FOLD) and
// computes this round's message in the same pass, so every live table entry is read once
// per round and the folded half is written once:
//   fold     u[j]  = t[2j] + r (t[2j+1] - t[2j])                    linear_prover.rs:151-178
//   message  s(c)  = sum_y prod_i (u_i[2y] + c (u_i[2y+1] - u_i[2y])),  c = 0..L   :82-140
// Sums of products are kept as unreduced 512-bit integers per thread (one Montgomery
// reduction per thread per evaluation point), then reduced over the warp by shuffles, over
// the block through shared memory and over the grid by the last block to finish.
#include "internal.hpp"
#include "reduce.cuh"
#include "round_pass.cuh"

namespace zk {

namespace {

constexpr int kThreads = kRoundThreads;
constexpr int kWarps = kRoundWarps;

template <int L>
struct RoundParams {
  const Fr* src[L];
  Fr* dst[L];
  FixedMul<FrParams> r;  // multiplier table of the challenge being bound
  uint64_t pairs;  // (even, odd) pairs of the table the message is computed over
  MsgSink sink;
};

template <int L, bool FOLD>
__global__ void __launch_bounds__(kThreads, (L <= 1 ? 3 : 2)) k_round(const RoundParams<L> p) {
  __shared__ uint4 stage[kWarps][WarpTile<8>::kChunks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Fr s[L + 1];
  round_pass<L, FOLD>(p.src, p.dst, p.r, p.pairs, (uint64_t)blockIdx.x * kWarps + warp, (uint64_t)gridDim.x * kWarps,
                      stage[warp], lane, s);
  grid_sum<L + 1, kWarps>(s, p.sink);
}

// Last step of the protocol: bind the final challenge on the two remaining entries of each
// table and multiply the results (linear_prover.rs:181-190).  With bind == 0 the tables
// already hold one entry each (num_var == 0).
struct FinalParams {
  const Fr* src[kMaxPolys];
  int num_poly;
  int bind;
  Fr r;
  Fr* out;  // out[0..num_poly) = a_arrays[i][0], out[num_poly] = product
};

__global__ void k_final(const FinalParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  Fr prod = Fr::one();
  for (int i = 0; i < p.num_poly; i++) {
    Fr a = p.src[i][0];
    if (p.bind) a = add(a, mul(p.r, sub(p.src[i][1], a)));
    p.out[i] = a;
    prod = mul(prod, a);
  }
  p.out[p.num_poly] = prod;
}

// Plain fold of the lowest variable (no message): util/poly.rs:852-884.
struct FoldParams {
  const Fr* src;
  Fr* dst;
  FixedMul<FrParams> r;
  uint64_t out_len;
};

__global__ void __launch_bounds__(kThreads) k_fold(const FoldParams p) {
  __shared__ uint4 stage[kWarps][WarpTile<4>::kChunks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4* sw = stage[warp];
  const uint64_t tiles = (p.out_len + 31) >> 5;
  for (uint64_t tile = (uint64_t)blockIdx.x * kWarps + warp; tile < tiles; tile += (uint64_t)gridDim.x * kWarps) {
    const uint64_t e0 = tile << 5;
    const uint32_t valid = (uint32_t)((p.out_len - e0) < 32 ? (p.out_len - e0) : 32);
    uint4 raw[4], q[4];
    WarpTile<4>::issue(reinterpret_cast<const uint4*>(p.src) + e0 * 4, valid * 4, lane, raw);
    WarpTile<4>::transpose_in(sw, lane, raw, q);
    const Fr a = fr_from_chunks(q[0], q[1]), b = fr_from_chunks(q[2], q[3]);
    const Fr u = add(a, mul_fixed(p.r, sub(b, a)));
    uint4 o[2];
    fr_to_chunks(u, o[0], o[1]);
    WarpTile<2>::store(reinterpret_cast<uint4*>(p.dst) + e0 * 2, valid * 2, sw, lane, o);
  }
}

// Two folds in one pass (challenges r0 then r1): dst[y] from src[4y .. 4y+3].  Used when the
// first of the two folds could be postponed, so the table is read once for both.
struct Fold2Params {
  const Fr* src;
  Fr* dst;
  FixedMul<FrParams> r0, r1, r01;  // r01 = r0 * r1
  uint64_t out_len;
};

__global__ void __launch_bounds__(kThreads) k_fold2(const Fold2Params p) {
  // two input stages per warp: the next tile streams in (cp.async) while this one is folded
  __shared__ uint4 stage[2][kWarps][WarpTile<8>::kChunks];
  __shared__ uint4 out_stage[kWarps][WarpTile<2>::kChunks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t tiles = (p.out_len + 31) >> 5;
  const uint64_t stride = (uint64_t)gridDim.x * kWarps;
  const uint4* src = reinterpret_cast<const uint4*>(p.src);
  auto valid_of = [&](uint64_t tile) { return (uint32_t)((p.out_len - (tile << 5)) < 32 ? (p.out_len - (tile << 5)) : 32); };
  uint64_t tile = (uint64_t)blockIdx.x * kWarps + warp;
  int buf = 0;
  if (tile < tiles) WarpTile<8>::prefetch_async(stage[0][warp], src + (tile << 5) * 8, valid_of(tile) * 8, lane);
  for (; tile < tiles; tile += stride, buf ^= 1) {
    const uint64_t e0 = tile << 5;
    const uint32_t valid = valid_of(tile);
    const uint64_t next = tile + stride;
    if (next < tiles) {
      WarpTile<8>::prefetch_async(stage[buf ^ 1][warp], src + (next << 5) * 8, valid_of(next) * 8, lane);
      WarpTile<8>::wait_async<1>();
    } else {
      WarpTile<8>::wait_async<0>();
    }
    uint4 q[8];
    WarpTile<8>::read_rows(stage[buf][warp], lane, q);
    const Fr t0 = fr_from_chunks(q[0], q[1]), t1 = fr_from_chunks(q[2], q[3]);
    const Fr t2 = fr_from_chunks(q[4], q[5]), t3 = fr_from_chunks(q[6], q[7]);
    // (t0 + r0 d01) + r1 ((t2 + r0 d23) - (t0 + r0 d01)) = t0 + r0 d01 + r1 (t2 - t0) + r0 r1 (d23 - d01)
    uint32_t d01[8], d02[8], d23[8], dd[8], m2[8], tmp[8];
    sub_lazy<FrParams>(d01, t1, t0);
    sub_lazy<FrParams>(d02, t2, t0);
    sub_lazy<FrParams>(d23, t3, t2);
#pragma unroll
    for (int i = 0; i < 8; i++) m2[i] = FrParams::mod(i);
    (void)add8(tmp, d23, m2);  // d23 + 2p - d01 stays below 4p < 2^256
    (void)add8(tmp, tmp, m2);
    (void)sub8(dd, tmp, d01);
    const Fr u = add(t0, mul_fixed3(p.r0, d01, p.r1, d02, p.r01, dd));
    uint4 o[2];
    fr_to_chunks(u, o[0], o[1]);
    WarpTile<2>::store(reinterpret_cast<uint4*>(p.dst) + e0 * 2, valid * 2, out_stage[warp], lane, o);
  }
}

int grid_for(uint64_t tiles, int max_blocks) {
  uint64_t blocks = (tiles + kWarps - 1) / kWarps;
  if (blocks < 1) blocks = 1;
  if (blocks > (uint64_t)max_blocks) blocks = max_blocks;
  return (int)blocks;
}

template <int L>
void launch_round_t(bool fold, const Fr* const* src, Fr* const* dst, const Fr& r, uint64_t pairs,
                    const RoundScratch& sc, cudaStream_t stream) {
  RoundParams<L> p;
  for (int i = 0; i < L; i++) {
    p.src[i] = src[i];
    p.dst[i] = fold ? dst[i] : nullptr;
  }
  p.r = make_fixed_mul(r);
  p.pairs = pairs;
  p.sink = sc.sink;
  static int occ[2] = {0, 0};  // resident blocks per SM, per variant
  if (!occ[fold]) {
    int o = 0;
    if (fold)
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, k_round<L, true>, kThreads, 0);
    else
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, k_round<L, false>, kThreads, 0);
    occ[fold] = o > 0 ? o : 1;
  }
  int cap = sc.sm_count * occ[fold];
  if (cap > sc.max_blocks) cap = sc.max_blocks;
  const int grid = grid_for((pairs + 31) / 32, cap);
  if (fold)
    k_round<L, true><<<grid, kThreads, 0, stream>>>(p);
  else
    k_round<L, false><<<grid, kThreads, 0, stream>>>(p);
}

}  // namespace

void launch_round(int num_poly, bool fold, const Fr* const* src, Fr* const* dst, const Fr& r, uint64_t pairs,
                  const RoundScratch& sc, cudaStream_t stream) {
  switch (num_poly) {
    case 1: launch_round_t<1>(fold, src, dst, r, pairs, sc, stream); break;
    case 2: launch_round_t<2>(fold, src, dst, r, pairs, sc, stream); break;
    case 3: launch_round_t<3>(fold, src, dst, r, pairs, sc, stream); break;
    case 4: launch_round_t<4>(fold, src, dst, r, pairs, sc, stream); break;
    default: break;  // callers check 1 <= num_poly <= kMaxPolys
  }
}

void launch_final(int num_poly, bool bind, const Fr* const* src, const Fr& r, Fr* out, cudaStream_t stream) {
  FinalParams p;
  for (int i = 0; i < kMaxPolys; i++) p.src[i] = i < num_poly ? src[i] : nullptr;
  p.num_poly = num_poly;
  p.bind = bind ? 1 : 0;
  p.r = r;
  p.out = out;
  k_final<<<1, 32, 0, stream>>>(p);
}

void launch_fold(const Fr* src, Fr* dst, const Fr& r, uint64_t out_len, int max_blocks, cudaStream_t stream) {
  FoldParams p{src, dst, make_fixed_mul(r), out_len};
  k_fold<<<grid_for((out_len + 31) / 32, max_blocks), kThreads, 0, stream>>>(p);
}

void launch_fold2(const Fr* src, Fr* dst, const Fr& r0, const Fr& r1, uint64_t out_len, int max_blocks,
                  cudaStream_t stream) {
  Fold2Params p{src, dst, make_fixed_mul(r0), make_fixed_mul(r1), make_fixed_mul(mul(r0, r1)), out_len};
  k_fold2<<<grid_for((out_len + 31) / 32, max_blocks), kThreads, 0, stream>>>(p);
}

}  // namespace zk
