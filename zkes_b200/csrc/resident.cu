// Several rounds of the dense prover in one cooperative launch.
//
// With the built-in transcript nothing of a round has to leave the device.  The launch is cooperative so that
// all blocks are resident together; every wait is bounded and reports through ResidentShared::error instead of
// spinning on.  Rounds: linear_prover.rs:59-72; message :82-140; fold :151-178; final :181-190.
//
// Large tables, rounds "in step": every block folds and sums its share of the tables and adds it to the round's
// accumulators (atomic additions of 64-bit limb sums, no modular arithmetic); block 0 waits until all have arrived,
// reduces the sums, runs the Fiat-Shamir step (one warp, transcript.rs:27-42 over STROBE / Keccak-f; the state
// stays in that warp's registers for the whole launch) and hands the challenge out as a tagged element; every block
// builds the challenge's multiplier table from it (one product) and starts the next round.  Waits are polled by a
// whole warp in lockstep: a warp that leaves a single-lane polling loop stays split and runs the code after it
// several times slower.
//
// Small tables, rounds "ahead" (ahead_rounds below): a round is then all latency - a dependent field product
// takes about 0.5 us, the transcript step 5 us, a hand-over between blocks 0.5 us - and in step these add up.
// Block 0 does nothing but the transcript chain, and the other blocks prepare message t + 1 while r_t is still
// being hashed: folding by r_t is linear in r_t, so message t + 1 is a polynomial of degree L in r_t,
//     s_{t+1}(c) = G(c, r_t),   G(c, rho) = sum_y prod_i bilinear(T_i[4y .. 4y+3]; rho, c),
// the round polynomial of two variables at once.  The workers tabulate G on {0..L}^2 right after the fold that
// produced the tables; block 0 interpolates the message when r_t is out (one product deep) and goes straight on to
// hash it.  Every value is an exact field element, so the messages are the reference's, bit for bit.  This mode
// runs to the end of the protocol, final values included.
#include <cstring>
#include "internal.hpp"
#include "round_pass.cuh"
#include "strobe_dev.cuh"

namespace zk {
namespace {

constexpr int kThreads = kRoundThreads;
constexpr int kWarps = kRoundWarps;
static_assert(sizeof(ResidentShared) <= 8192, "the context allocates 8192 bytes for the hand-over area");

template <int L>
struct ResidentParams {
  const Fr* src[L];
  Fr* ping[L];
  Fr* pong[L];
  uint64_t size;        // entries per table on entry (a power of two, at least 4)
  uint32_t rounds;      // messages to produce
  uint32_t spin_limit;  // polls before a wait gives up
  uint32_t pending;     // non-zero: no round in step; the tables are entered with sh->challenge still to be bound (as if
                        // round 0 had been done elsewhere), ahead_from = 1, and sh->st holds the transcript state
  uint32_t ahead_from;  // first round whose message is prepared ahead of its challenge; >= rounds: none, and the
                        // last challenge is left unbound.  Otherwise 1 <= ahead_from < rounds, rounds = log2(size),
                        // and the launch also binds the last challenge and writes the final values.
  StrobeState st;       // transcript state on entry
  Fr* partials;         // gridDim.x * (L + 1)
  ResidentShared* sh;   // zeroed on entry
  Fr* out_msgs;         // rounds * (L + 1), canonical integers (not Montgomery form)
  Fr* out_chal;         // rounds, canonical integers
  Fr* out_final;        // rounds ahead: the L table values at the challenge point, then their product
  StrobeState* out_st;  // rounds ahead: transcript state after the last challenge
  Fr pow2[8];           // 2^(32 j + 64) mod r in Montgomery form: times a canonical challenge, the rows of its multiplier table
  Fr kconst[L + 1];     // R^(L+1) / prod_{k != j} (j - k) as integers: scales the grid sums for the interpolation
  PeerExchange px;      // px.world > 1: sharded instance, messages are summed over the ranks
};


// Field products outside the streaming passes are called, not inlined: a product is about 3.5 KB of code, the
// rounds of small tables run each piece of code once per round, and what bounds them then is fetching
// instructions, not executing them.  One shared copy stays in the instruction cache.
__device__ __noinline__ Fr mul_call(Fr a, Fr b) { return mul(a, b); }
__device__ __forceinline__ Fr to_mont_call(const Fr& a) { return mul_call(Fr::r2(), a); }

// Bounded wait for a counter to reach `want`; false when it gave up (or another block did).  Called by all the
// lanes of a warp together, which then poll in lockstep (one transaction per poll): with a single lane in the
// loop the warp stayed split after the wait and ran what followed - the transcript step - several times slower.
__device__ __forceinline__ bool wait_counter(const unsigned int* counter, unsigned int want, unsigned int* error, uint32_t limit) {
  const volatile unsigned int* c = reinterpret_cast<const volatile unsigned int*>(counter);
  const volatile unsigned int* err = reinterpret_cast<const volatile unsigned int*>(error);
  uint32_t polls = 0;
  bool ok = true;
  while (true) {
    // lane 0's reading decides for the warp, so that the lanes leave the loop together
    const unsigned int v = __shfl_sync(0xffffffffu, *c, 0), e = __shfl_sync(0xffffffffu, *err, 0);
    if (v >= want) break;
    if (e != 0) {  // another block gave up and said why: leave its code in place
      ok = false;
      break;
    }
    if (++polls > limit) {
      if ((threadIdx.x & 31) == 0) atomicCAS(error, 0u, 1u);
      ok = false;
      break;
    }
    __nanosleep(40);  // a pause that leaves the issue slots to the block this SM may share with
  }
  __threadfence();
  return ok;
}

__device__ __forceinline__ Fr shfl_xor_fr(const Fr& x, int mask) {
  Fr r;
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = __shfl_xor_sync(0xffffffffu, x.v[i], mask);
  return r;
}

// Chunk `part` (0..2) of a tagged element.
__device__ __forceinline__ void st_tagged_part(TaggedFr* dst, const Fr& x, uint32_t tag, int part) {
  const uint32_t a = x.v[3 * part], b = x.v[3 * part + 1], c = part < 2 ? x.v[3 * part + 2] : 0u;
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(&dst->w[part][0]), "r"(a), "r"(b), "r"(c), "r"(tag) : "memory");
}
__device__ __forceinline__ void st_tagged(TaggedFr* dst, const Fr& x, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(&dst->w[0][0]), "r"(x.v[0]), "r"(x.v[1]), "r"(x.v[2]), "r"(tag) : "memory");
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(&dst->w[1][0]), "r"(x.v[3]), "r"(x.v[4]), "r"(x.v[5]), "r"(tag) : "memory");
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(&dst->w[2][0]), "r"(x.v[6]), "r"(x.v[7]), "r"(0u), "r"(tag) : "memory");
}
// One reading of a tagged element: true when all three chunks carry `tag` (then `out` is the element).
__device__ __forceinline__ bool ld_tagged(const TaggedFr* src, uint32_t tag, Fr& out) {
  uint32_t t0, t1, t2, z;
  (void)z;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(out.v[0]), "=r"(out.v[1]), "=r"(out.v[2]), "=r"(t0) : "l"(&src->w[0][0]) : "memory");
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(out.v[3]), "=r"(out.v[4]), "=r"(out.v[5]), "=r"(t1) : "l"(&src->w[1][0]) : "memory");
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(out.v[6]), "=r"(out.v[7]), "=r"(z), "=r"(t2) : "l"(&src->w[2][0]) : "memory");
  return t0 == tag && t1 == tag && t2 == tag;
}
// Bounded wait of a whole warp for tagged elements: lanes with `mine` poll their own element, the others go along;
// the lanes leave the loop together.  false when it gave up (or another block did).
__device__ __forceinline__ bool wait_tagged(const TaggedFr* src, bool mine, uint32_t tag, Fr& out, unsigned int* error, uint32_t limit) {
  const volatile unsigned int* err = reinterpret_cast<const volatile unsigned int*>(error);
  uint32_t polls = 0;
  while (true) {
    const bool have = !mine || ld_tagged(src, tag, out);
    if (__all_sync(0xffffffffu, have)) return true;
    if (__shfl_sync(0xffffffffu, *err, 0) != 0) return false;  // another block gave up and said why
    if (++polls > limit) {
      if ((threadIdx.x & 31) == 0) atomicCAS(error, 0u, 1u);
      return false;
    }
    __nanosleep(40);  // a pause that leaves the issue slots to the block this SM may share with
  }
}

// a + k (b - a) for k in 0 .. 3 (additions only).
__device__ __forceinline__ Fr lin_small(const Fr& a, const Fr& b, int k) {
  if (k == 0) return a;
  if (k == 1) return b;
  const Fr d = sub(b, a);
  Fr r = b;
  for (int i = 1; i < k; i++) r = add(r, d);
  return r;
}

// x mod r for any 256-bit x (x < 6 r).
__device__ __forceinline__ Fr reduce_256(const Fr& x) {
  Fr r = x;
#pragma unroll
  for (int sh = 2; sh >= 0; sh--) {  // 4 r, 2 r, r
    uint32_t m[8], d[8];
#pragma unroll
    for (int i = 0; i < 8; i++)
      m[i] = (FrParams::mod(i) << sh) | (sh && i ? FrParams::mod(i - 1) >> (32 - sh) : 0u);
    const uint32_t borrow = sub8(d, r.v, m);
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = borrow ? r.v[i] : d[i];
  }
  return r;
}

// How a warp of a worker block splits a unit of the rounds ahead.  A unit is QW quads of the folded tables
// (four consecutive entries each).  Lane = ql * LQ + e * LT + ts: quad ql of the unit, entry e of the quad, table
// slot ts.  Fold: lanes with ts < L bind the challenge on their entry (one product).  Grid: the (L + 1)^2 points
// of a quad are dealt to its LQ lanes, point pt = w + k * LQ to lane w = e * LT + ts (L - 1 products each).  Two
// tables get four slots as well: sixteen lanes then take the nine points one each, which is a product less on the
// way from the challenge to the next message than eight lanes with two points on one of them.
template <int L>
struct AheadSplit {
  static constexpr int NV = L + 1, NG = NV * NV;
  static constexpr int LT = L == 1 ? 1 : 4;
  static constexpr int LQ = 4 * LT;
  static constexpr int QW = 32 / LQ;
  static constexpr int PL = (NG + LQ - 1) / LQ;
};

// The rounds from p.ahead_from to the end.  Entered by every block right after its part of the in-step round
// ahead_from - 1 (block 0: after that round's transcript step, with the state in `ws`): the tables `cur` (cur_size
// entries) are the ones message ahead_from - 1 is over, complete once every block has arrived at that round's
// ticket, and the challenge of that round arrives as rplain[(ahead_from - 1) & 1].
template <int L>
__device__ __forceinline__ void ahead_rounds(const ResidentParams<L>& p, WarpStrobe& ws, const Fr* (&cur)[L], uint64_t cur_size,
                                             uint8_t* stream, int* ok_flag, int* flag) {
  using S = AheadSplit<L>;
  constexpr int NV = S::NV, NG = S::NG, LT = S::LT, LQ = S::LQ, QW = S::QW, PL = S::PL;
  __shared__ Fr xch[kWarps][32];
  __shared__ Fr red[kWarps][NG];
  __shared__ unsigned long long limbs[NG][8];
  __shared__ Fr lag[NG];
  __shared__ Fr r_sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t t0 = p.ahead_from;
  ResidentShared* sh = p.sh;

  if (blockIdx.x == 0) {
    // ------------------------------------------------------------------ the transcript chain (one warp)
    if (warp != 0) return;
    Fr r = Fr::zero();  // the challenge of the round before, canonical; the transcript state is in this warp's registers
    if (!wait_tagged(&sh->rplain[(t0 - 1) & 1], true, t0, r, &sh->error, p.spin_limit)) return;
    const int j = lane % NV;
    for (uint32_t t = t0; t < p.rounds; t++) {
      // lambda'_j = prod_{k != j} (r - k) / R^(L-1); the grid sums arrive scaled by R^L / prod_{k != j} (j - k)
      // (the L nodes other than j, in the same order of operations in every lane: one product sequence per warp)
      Fr lam;
#pragma unroll
      for (int m = 0; m < L; m++) {
        Fr kk = Fr::zero();
        kk.v[0] = (uint32_t)(m < j ? m : m + 1);
        const Fr term = sub(r, kk);
        lam = m == 0 ? term : mul_call(lam, term);
      }
      Fr g = Fr::zero();
      if (!wait_tagged(&sh->gsum[t & 1][lane < NG ? lane : 0], lane < NG, t + 1, g, &sh->error, p.spin_limit)) return;
      if (lane < NG) lag[lane] = mul_call(lam, g);  // lane = c * NV + j
      __syncwarp();
      if (lane < NV) {  // s_t(c), canonical
        Fr s = lag[lane * NV];
#pragma unroll
        for (int k = 1; k < NV; k++) s = add(s, lag[lane * NV + k]);
        p.out_msgs[(size_t)t * NV + lane] = s;
        uint8_t* dst = WarpStrobe::round_stream_data(stream, lane);
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
          for (int k = 0; k < 4; k++) dst[4 * i + k] = (uint8_t)(s.v[i] >> (8 * k));
      }
      __syncwarp();
      Fr raw;
      ws.fs_round<L>(stream, lane, raw.v);
      r = reduce_256(raw);
      if (lane < 3) st_tagged_part(&sh->rplain[t & 1], r, t + 1, lane);  // the hand-over to the workers
      if (lane == 0) p.out_chal[t] = r;
    }
    if (lane < 25) p.out_st->lanes[lane] = ws.a;
    if (lane == 0) {
      p.out_st->pos = ws.pos;
      p.out_st->pos_begin = ws.pos_begin;
      p.out_st->cur_flags = 1u | 2u | 4u;
      p.out_st->pad = 0;
    }
    return;
  }

  // -------------------------------------------------------------------- workers
  const uint32_t nbw = gridDim.x - 1;                      // worker blocks
  const uint64_t wid = (blockIdx.x - 1) + (uint64_t)nbw * warp;  // consecutive units go to different SMs first
  const uint64_t wtotal = (uint64_t)nbw * kWarps;
  const int ql = lane / LQ, w = lane % LQ, e = w / LT, ts = w % LT;
  unsigned int tickets = 0;  // arrivals expected so far at sh->garrive (the same in every block that is still here)
  Fr r_mont = Fr::zero();
  // pass `it` = t0 - 1: the grid of message t0 over the tables as they are.  Pass it >= t0: bind r_{it-1}, which
  // gives the tables of message `it`, then the grid of message it + 1 over them (none after the last message).
  for (uint32_t it = t0 - 1; it < p.rounds; it++) {
    const bool do_fold = it >= t0, do_grid = it + 1 < p.rounds;
    const uint64_t e_out = do_fold ? cur_size >> 1 : cur_size;  // entries of the tables this pass leaves
    const uint64_t n_q = e_out >> 2;
    const uint64_t n_units = n_q ? (n_q + QW - 1) / QW : 1;
    if (blockIdx.x - 1 >= n_units) return;  // no unit in this pass, and none in any later one
    const unsigned int active = (unsigned int)(n_units < nbw ? n_units : nbw);
    Fr* dst[L];
#pragma unroll
    for (int i = 0; i < L; i++) dst[i] = (it & 1) ? p.ping[i] : p.pong[i];
    const Fr* my_src = cur[0];  // the table of this lane's slot
    Fr* my_dst = dst[0];
#pragma unroll
    for (int i = 1; i < L; i++) {
      if (ts == i) {
        my_src = cur[i];
        my_dst = dst[i];
      }
    }
    {  // what this pass reads is complete in every block: the tables of the last round in step (every block has
       // arrived there), or those of the pass before, whose tickets are then all in as well
      if (warp == 0) {
        const bool ok = it >= t0 ? wait_counter(&sh->gseq, it + 1, &sh->error, p.spin_limit)
                                 : wait_counter(&sh->arrive, t0 * gridDim.x, &sh->error, p.spin_limit);
        if (lane == 0) *ok_flag = ok ? 1 : 0;
      }
      __syncthreads();
      if (!*ok_flag) return;
    }
    // the first unit's entries do not depend on the challenge: fetch them before waiting for it
    uint64_t u = wid;
    Fr a0 = Fr::zero(), a1 = Fr::zero();
    auto fetch = [&](uint64_t unit) {
      const uint64_t i = 4 * (unit * QW + ql) + e;
      if (ts < L && i < e_out) {
        if (do_fold) {
          a0 = ld_cg_fr(my_src + 2 * i);
          a1 = ld_cg_fr(my_src + 2 * i + 1);
        } else {
          a0 = ld_cg_fr(my_src + i);
        }
      }
    };
    if (u < n_units) fetch(u);
    if (it >= t0) {
      __syncthreads();  // ok_flag is free again
      if (warp == 0) {
        Fr rp = Fr::zero();
        const bool ok = wait_tagged(&sh->rplain[(it - 1) & 1], true, it, rp, &sh->error, p.spin_limit);
        if (lane == 0) {
          *ok_flag = ok ? 1 : 0;
          r_sm = rp;
        }
      }
      __syncthreads();
      if (!*ok_flag) return;
      r_mont = to_mont_call(r_sm);
    }
    Fr acc[PL];
#pragma unroll
    for (int k = 0; k < PL; k++) acc[k] = Fr::zero();
    for (; u < n_units; u += wtotal) {
      if (u != wid) fetch(u);
      const uint64_t q = u * QW + ql, i = 4 * q + e;
      const bool ent_ok = ts < L && i < e_out;
      Fr v = a0;
      if (do_fold) {
        v = add(a0, mul_call(r_mont, sub(a1, a0)));
        if (ent_ok) my_dst[i] = v;
      }
      xch[warp][lane] = ent_ok ? v : Fr::zero();
      __syncwarp();
      if (do_grid && q < n_q) {
        const Fr* quad = &xch[warp][ql * LQ];  // entry e', table t' at [e' * LT + t']
#pragma unroll
        for (int k = 0; k < PL; k++) {
          const int pt = w + k * LQ;
          if (pt < NG) {
            const int c = pt / NV, rho = pt % NV;
            Fr prod;
#pragma unroll
            for (int t = 0; t < L; t++) {
              const Fr e0 = lin_small(quad[0 * LT + t], quad[1 * LT + t], rho);
              const Fr e1 = lin_small(quad[2 * LT + t], quad[3 * LT + t], rho);
              const Fr x = lin_small(e0, e1, c);
              prod = t == 0 ? x : mul_call(prod, x);
            }
            acc[k] = add(acc[k], prod);
          }
        }
      }
      __syncwarp();
    }
    if (do_grid) {
      // lanes of equal role over the quads of the warp, then the warps of the block as plain 64-bit limb sums,
      // then the blocks by atomic additions of those limbs: no modular arithmetic until the very end
#pragma unroll
      for (int k = 0; k < PL; k++) {
#pragma unroll
        for (int off = LQ; off < 32; off <<= 1) acc[k] = add(acc[k], shfl_xor_fr(acc[k], off));
        const int pt = w + k * LQ;
        if (ql == 0 && pt < NG) red[warp][pt] = acc[k];
      }
      __syncthreads();
      const int par = (it + 1) & 1;
      if (threadIdx.x < NG * 8) {
        const int pt = threadIdx.x >> 3, limb = threadIdx.x & 7;
        unsigned long long s = 0;
#pragma unroll
        for (int ww = 0; ww < kWarps; ww++)
          if ((blockIdx.x - 1) + (uint64_t)nbw * ww < n_units) s += red[ww][pt].v[limb];
        atomicAdd(&sh->gacc[par][pt][limb], s);
      }
      __threadfence();  // this block's folded entries and its share of the grid, before the ticket
      __syncthreads();
      tickets += active;
      if (threadIdx.x == 0) *flag = atomicAdd(&sh->garrive, 1u) == tickets - 1;
      __syncthreads();
      if (*flag) {
        __threadfence();
        if (threadIdx.x < NG * 8) {
          const int pt = threadIdx.x >> 3, limb = threadIdx.x & 7;
          limbs[pt][limb] = atomicExch(&sh->gacc[par][pt][limb], 0ull);  // read, and cleared for the pass after the next
        }
        __syncthreads();
        if (threadIdx.x < NG) {
          Wide x;
#pragma unroll
          for (int k = 0; k < 16; k++) x.v[k] = 0;
          unsigned long long carry = 0;
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const unsigned long long v = limbs[threadIdx.x][k];
            const unsigned long long s = (v & 0xffffffffull) + (carry & 0xffffffffull);
            x.v[k] = (uint32_t)s;
            carry = (v >> 32) + (carry >> 32) + (s >> 32);
          }
          x.v[8] = (uint32_t)carry;
          x.v[9] = (uint32_t)(carry >> 32);
          // the sum of Montgomery forms is G R as an integer: / R, then the constant of this point's column
          Fr kc = p.kconst[0];
#pragma unroll
          for (int k = 1; k < NV; k++)
            if ((int)(threadIdx.x % NV) == k) kc = p.kconst[k];
          st_tagged(&sh->gsum[par][threadIdx.x], mul_call(redc<FrParams>(x), kc), it + 2);  // to the transcript block
        }
        // to the workers: the fence after the ticket orders every block's entries before this store
        if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(&sh->gseq) = it + 2;
      }
    } else {
      __syncthreads();
    }
    if (do_fold) {
#pragma unroll
      for (int i = 0; i < L; i++) cur[i] = dst[i];
      cur_size >>= 1;
    }
  }
  // The last pass left two entries per table, folded by unit 0 = this block's warp 0 (block 1 only gets here with
  // a unit; the others have left), still in its exchange buffer.  Bind the last challenge.
  if (blockIdx.x != 1 || warp != 0) return;
  Fr rp = Fr::zero();
  if (!wait_tagged(&sh->rplain[(p.rounds - 1) & 1], true, p.rounds, rp, &sh->error, p.spin_limit)) return;
  r_mont = to_mont_call(rp);
  if (lane < L) {
    const Fr b0 = xch[0][0 * LT + lane], b1 = xch[0][1 * LT + lane];
    const Fr f = add(b0, mul_call(r_mont, sub(b1, b0)));
    p.out_final[lane] = f;
    lag[lane] = f;
  }
  __syncwarp();
  if (lane == 0) {
    Fr prod = lag[0];
#pragma unroll
    for (int t = 1; t < L; t++) prod = mul_call(prod, lag[t]);
    p.out_final[L] = prod;
  }
}

template <int L>
__global__ void __launch_bounds__(kThreads, (L <= 1 ? 3 : 2)) k_resident(const ResidentParams<L> p) {
  extern __shared__ uint4 resident_stage[];  // per warp: 2 stages x L tables of WarpTile<8>::kChunks slots
  uint4* const my_stage = resident_stage + (size_t)(threadIdx.x >> 5) * (2 * L * WarpTile<8>::kChunks);
  __shared__ FixedMul<FrParams> r_tab;
  __shared__ Fr red[kWarps][L + 1];
  __shared__ Fr msg[L + 1];
  __shared__ __align__(16) uint8_t stream[WarpStrobe::round_stream_bytes<L>() + 15];
  __shared__ unsigned long long macc_sm[L + 1][8];
  __shared__ int flag, ok_flag, px_ok;
  __shared__ uint32_t px_stage[kPeerRanks * (L + 1) * 8];
  __shared__ __align__(16) uint64_t keccak_scratch[64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int NV = L + 1;
  if (threadIdx.x == 0) WarpStrobe::init_round_stream<L>(stream);

  WarpStrobe ws;  // the transcript: block 0, warp 0
  ws.scratch = keccak_scratch;
  ws.a = lane < 25 ? p.st.lanes[lane] : 0;
  ws.pos = p.st.pos;
  ws.pos_begin = p.st.pos_begin;
  const Fr* cur[L];
#pragma unroll
  for (int i = 0; i < L; i++) cur[i] = p.src[i];
  uint64_t cur_size = p.size;
  // consecutive tiles go to different blocks first, so that a small table spreads over the SMs
  const uint64_t warp_global = blockIdx.x + (uint64_t)gridDim.x * warp, warp_stride = (uint64_t)gridDim.x * kWarps;

  if (p.pending) {
    if constexpr (L <= 3) {
      if (threadIdx.x == 0) atomicAdd(&p.sh->arrive, 1u);  // stands for the ticket of the round that was done elsewhere
      if (blockIdx.x == 0 && warp == 0) {
        ws.a = lane < 25 ? p.sh->st.lanes[lane] : 0;
        ws.pos = p.sh->st.pos;
        ws.pos_begin = p.sh->st.pos_begin;
        Fr one_plain = Fr::zero();
        one_plain.v[0] = 1;
        const Fr rc = mul_call(p.sh->challenge, one_plain);  // out of Montgomery form
        if (lane < 3) st_tagged_part(&p.sh->rplain[0], rc, 1, lane);
      }
      ahead_rounds<L>(p, ws, cur, cur_size, stream, &ok_flag, &flag);
    }
    return;
  }
  for (uint32_t round = 0; round < p.rounds; round++) {
    Fr s[NV];
    if (round == 0) {
      round_pass_async<L, false>(cur, cur, r_tab, cur_size >> 1, warp_global, warp_stride, my_stage, lane, s);
    } else {
      Fr* dst[L];
#pragma unroll
      for (int i = 0; i < L; i++) dst[i] = (round & 1) ? p.ping[i] : p.pong[i];
      round_pass_async<L, true>(cur, dst, r_tab, cur_size >> 2, warp_global, warp_stride, my_stage, lane, s);
#pragma unroll
      for (int i = 0; i < L; i++) cur[i] = dst[i];
      cur_size >>= 1;
    }
    // Block total -> global: the warps' sums are added as plain 64-bit sums of their 32-bit limbs, and the blocks add
    // those to the round's accumulators by atomics, so nobody has to read a partial sum per block afterwards.
    const uint64_t tiles = ((cur_size >> 1) + 31) >> 5;  // cur_size: entries of the table the message is over
    const int mpar = round & 1;
    if (blockIdx.x < tiles) {  // the others had no tile this round
#pragma unroll
      for (int c = 0; c < NV; c++) {
        const Fr t = warp_sum(s[c]);
        if (lane == 0) red[warp][c] = t;
      }
      __syncthreads();
      if (threadIdx.x < NV * 8) {
        const int c = threadIdx.x >> 3, limb = threadIdx.x & 7;
        unsigned long long v = 0;
#pragma unroll
        for (int w = 0; w < kWarps; w++)
          if (blockIdx.x + (uint64_t)gridDim.x * w < tiles) v += red[w][c].v[limb];
        atomicAdd(&p.sh->macc[mpar][c][limb], v);
      }
      __threadfence();  // this block's folded entries and its share, before the ticket
    }
    __syncthreads();
    // Block 0 owns the rest of every round: it waits until all blocks have arrived.  (The last block to arrive
    // could go on at once, but it is a different block, on a different SM, every round, and the code of the
    // transcript step is then fetched anew: that cost more than this hand-over.)
    if (threadIdx.x == 0) atomicAdd(&p.sh->arrive, 1u);
    if (blockIdx.x == 0) {
      if (warp == 0) {
        const bool ok = wait_counter(&p.sh->arrive, (round + 1) * gridDim.x, &p.sh->error, p.spin_limit);
        if (lane == 0) ok_flag = ok ? 1 : 0;
      }
      __syncthreads();
      if (!ok_flag) return;
    }
    if (blockIdx.x == 0) {
      if (threadIdx.x < NV * 8) {  // read, and cleared for the round after the next
        const int c = threadIdx.x >> 3, limb = threadIdx.x & 7;
        macc_sm[c][limb] = atomicExch(&p.sh->macc[mpar][c][limb], 0ull);
      }
      __syncthreads();
      if (threadIdx.x < NV) {
        Wide x;
#pragma unroll
        for (int k = 0; k < 16; k++) x.v[k] = 0;
        unsigned long long carry = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
          const unsigned long long v = macc_sm[threadIdx.x][k];
          const unsigned long long lo = (v & 0xffffffffull) + (carry & 0xffffffffull);
          x.v[k] = (uint32_t)lo;
          carry = (v >> 32) + (carry >> 32) + (lo >> 32);
        }
        x.v[8] = (uint32_t)carry;
        x.v[9] = (uint32_t)(carry >> 32);
        msg[threadIdx.x] = redc<FrParams>(x);  // the sum of Montgomery forms, / R: the message as canonical integers
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
        if (lane <= L) {
          const Fr canon = msg[lane];
          p.out_msgs[(size_t)round * NV + lane] = canon;
          uint8_t* dst = WarpStrobe::round_stream_data(stream, lane);
#pragma unroll
          for (int i = 0; i < 8; i++)
#pragma unroll
            for (int k = 0; k < 4; k++) dst[4 * i + k] = (uint8_t)(canon.v[i] >> (8 * k));
        }
        __syncwarp();
        Fr raw;
        ws.fs_round<L>(stream, lane, raw.v);
        const Fr r = reduce_256(raw);
        if (lane < 3) st_tagged_part(&p.sh->rplain[round & 1], r, round + 1, lane);  // the hand-over to every block
        if (lane == 0) p.out_chal[round] = r;
        if (round + 1 == p.rounds) {  // for the kernel that goes on: challenge in Montgomery form, transcript state
          if (lane < 25) p.sh->st.lanes[lane] = ws.a;
          if (lane == 0) {
            p.sh->challenge = to_mont_call(r);
            p.sh->st.pos = ws.pos;
            p.sh->st.pos_begin = ws.pos_begin;
            p.sh->st.cur_flags = 1u | 2u | 4u;
            p.sh->st.pad = 0;
          }
        }
      }
    }
    if (round + 1 == p.rounds) break;  // the last challenge is consumed by whoever runs next
    // wait for this round's challenge; every block builds the multiplier table from it by itself (one product)
    if (round + 1 == p.ahead_from) {  // the tables are small from here on
      if constexpr (L <= 3) ahead_rounds<L>(p, ws, cur, cur_size, stream, &ok_flag, &flag);
      return;
    }
    if (warp == 0) {
      Fr r = Fr::zero();
      const bool ok = wait_tagged(&p.sh->rplain[round & 1], true, round + 1, r, &p.sh->error, p.spin_limit);
      if (lane == 0) ok_flag = ok ? 1 : 0;
      if (ok && lane < 8) {  // row j = r 2^(32 j + 64) mod r as plain integers
        const Fr row = mul_call(r, p.pow2[lane]);
#pragma unroll
        for (int k = 0; k < 8; k++) r_tab.c[lane][k] = row.v[k];
      }
    }
    __syncthreads();
    if (!ok_flag) return;
  }
}

template <int L>
int launch_resident_t(const Fr* const* src, Fr* const* ping, Fr* const* pong, uint64_t size, uint32_t rounds,
                      const StrobeState& st, Fr* partials, int max_blocks, int sm_count, ResidentShared* sh, Fr* out_msgs,
                      Fr* out_chal, cudaStream_t stream, const PeerExchange* px, const ResidentToEnd* to_end) {
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
    p.pow2[j] = to_mont(cur);  // times a canonical challenge (Montgomery product): r 2^(32 j + 64) as a plain integer
    cur = mul(cur, step);
  }
  // the opt-in for more than 48 KB of dynamic shared memory is per device, and a process may hold contexts on several
  constexpr size_t kStageBytes = (size_t)kWarps * 2 * L * WarpTile<8>::kChunks * sizeof(uint4);
  if (cudaFuncSetAttribute(k_resident<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStageBytes) != cudaSuccess) return -2;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_resident<L>, kThreads, kStageBytes) != cudaSuccess || occ < 1) return -2;
  uint64_t grid = ((size >> 1) + 31) / 32;  // tiles of the first round, a warp each
  const uint64_t cap = (uint64_t)sm_count * occ < (uint64_t)max_blocks ? (uint64_t)sm_count * occ : (uint64_t)max_blocks;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  p.ahead_from = rounds;
  p.pending = 0;
  p.out_final = nullptr;
  p.out_st = nullptr;
  if (to_end) {
    // Rounds run ahead once the tables a grid pass reads have at most 2^ahead_log entries: message t is tabulated
    // over the tables of message t - 1 (size >> (t - 1) entries), at (L + 1)^2 products per four entries.  Needs
    // a block for the transcript beside at least one worker, a grid of at most kResidentGrid points, one GPU,
    // and all the rounds of the tables in this launch.
    if (px || L > 3 || cap < 2 || rounds < 2 || size != (1ull << rounds) || to_end->ahead_log < 2) return -5;
    // (a single table has no products in its grid, only additions: it can run ahead four times earlier)
    const uint32_t lg = to_end->ahead_log + (L == 1 ? 2 : 0);
    uint32_t t = 1;
    while (!to_end->pending && t + 1 < rounds && (size >> (t - 1)) > (1ull << lg)) t++;
    p.ahead_from = t;
    p.pending = to_end->pending ? 1u : 0u;
    // a block per unit of the first pass ahead (and the transcript block), so that the units spread over the SMs
    const uint64_t quads = (size >> (t - 1)) >> 2;
    const uint64_t units = quads ? (quads + AheadSplit<L < 4 ? L : 1>::QW - 1) / AheadSplit<L < 4 ? L : 1>::QW : 1;
    if (grid < units + 1) grid = units + 1 < cap ? units + 1 : cap;
    p.out_final = to_end->out_final;
    p.out_st = to_end->out_st;
    // host field inversions are slow (hundreds of products each): once per process and L
    struct Consts {
      Fr k[L + 1];
      Consts() {
        for (int j = 0; j <= L; j++) {
          Fr den = Fr::one();
          for (int i = 0; i <= L; i++) {
            if (i == j) continue;
            const Fr d = j > i ? from_u32<FrParams>((uint32_t)(j - i)) : neg(from_u32<FrParams>((uint32_t)(i - j)));
            den = mul(den, d);
          }
          Fr c = inverse(den);                          // R / den
          for (int i = 0; i < L; i++) c = to_mont(c);   // R^(L+1) / den
          k[j] = c;
        }
      }
    };
    static const Consts consts;
    for (int j = 0; j <= L; j++) p.kconst[j] = consts.k[j];
    *to_end->ahead_from = t;
  }
  void* args[] = {&p};
  // counters, tags and accumulators start from zero; a pending launch keeps the error word of the launch before
  // (its waits then give up at once) beside the challenge and the state that launch left
  if (p.pending) {
    if (cudaMemsetAsync(sh, 0, offsetof(ResidentShared, error), stream) != cudaSuccess) return -3;
    if (cudaMemsetAsync(&sh->garrive, 0, offsetof(ResidentShared, challenge) - offsetof(ResidentShared, garrive), stream) != cudaSuccess) return -3;
  } else if (cudaMemsetAsync(sh, 0, offsetof(ResidentShared, challenge), stream) != cudaSuccess) {
    return -3;
  }
  if (cudaLaunchCooperativeKernel((const void*)k_resident<L>, dim3((unsigned)grid), dim3(kThreads), args, kStageBytes, stream) !=
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
// launch was not possible and nothing ran.  With to_end (unsharded, at most three tables, rounds = log2(size) >= 2)
// the launch runs to the end of the protocol instead: the rounds from *to_end->ahead_from on are prepared ahead of
// their challenges, and the final values and the transcript state are written to to_end->out_final / out_st.
// Either way out_msgs and out_chal receive canonical integers, not Montgomery form.
int launch_resident(int num_poly, const Fr* const* src, Fr* const* ping, Fr* const* pong, uint64_t size, uint32_t rounds,
                    const StrobeState& st, Fr* partials, int max_blocks, int sm_count, ResidentShared* sh, Fr* out_msgs,
                    Fr* out_chal, cudaStream_t stream, const PeerExchange* px, const ResidentToEnd* to_end) {
  switch (num_poly) {
    case 1: return launch_resident_t<1>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px, to_end);
    case 2: return launch_resident_t<2>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px, to_end);
    case 3: return launch_resident_t<3>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px, to_end);
    case 4: return launch_resident_t<4>(src, ping, pong, size, rounds, st, partials, max_blocks, sm_count, sh, out_msgs, out_chal, stream, px, to_end);
    default: return -1;
  }
}

}  // namespace zk
