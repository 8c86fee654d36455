// Declarations shared by the kernels' translation units and the C ABI layer.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "ff.cuh"

namespace zk {

constexpr int kMaxPolys = 4;  // tables per product term the dense round kernel is built for

// Device scratch every round launch needs (owned by the context).
// Where a message kernel leaves its result.  The last block to finish writes the summed message
// to msg (device) and, when pub_flag is set, also to pub_msg in host-mapped memory followed by
// the launch's sequence number in pub_flag, which the host polls instead of synchronising.
struct MsgSink {
  Fr* partials;           // max_blocks * (kMaxPolys + 1) elements
  unsigned int* counter;  // zero between launches
  Fr* msg;                // up to 16 elements: the round message
  Fr* pub_msg;            // host-mapped copy of msg (device-visible address), or nullptr
  unsigned int* pub_flag; // host-mapped sequence word, or nullptr
  unsigned int seq;       // value to publish for this launch
};

struct RoundScratch {
  MsgSink sink;
  int max_blocks;         // capacity of sink.partials, in blocks
  int sm_count;
};

// sumcheck.cu
void launch_round(int num_poly, bool fold, const Fr* const* src, Fr* const* dst, const Fr& r, uint64_t pairs,
                  const RoundScratch& sc, cudaStream_t stream);
void launch_final(int num_poly, bool bind, const Fr* const* src, const Fr& r, Fr* out, cudaStream_t stream);
void launch_fold(const Fr* src, Fr* dst, const Fr& r, uint64_t out_len, int max_blocks, cudaStream_t stream);
void launch_fold2(const Fr* src, Fr* dst, const Fr& r0, const Fr& r1, uint64_t out_len, int max_blocks,
                  cudaStream_t stream);


// poly.cu
int launch_eq_table(const Fr* point_dev, const Fr* point_host, uint32_t k, Fr* out, int sm_count, cudaStream_t s);
void launch_dot(const Fr* a, const Fr* b, uint64_t n, const RoundScratch& sc, cudaStream_t s);
uint32_t from_right_splits(uint64_t lo_n, uint64_t hi_n, int sm_count);
int launch_from_right(const Fr* f, const Fr* eq, uint64_t lo_n, uint64_t hi_n, Fr* partial, Fr* out, int sm_count,
                      cudaStream_t s);

// intfold.cu
int launch_permute_ranges(const void* in, void* out, uint32_t n, uint32_t elem_bytes, const uint32_t* ranges,
                          uint32_t n_ranges, int sm_count, cudaStream_t s);
uint32_t int_fold_splits(uint64_t n_rows, uint64_t m_cols, int sm_count);
int launch_int_fold(const void* t, const Fr* eq, uint64_t n_rows, uint64_t m_cols, Fr* partial, Fr* out, int sm_count,
                    cudaStream_t s);

// general.cu
// eq: the plain table when `ones` (first round, every value one), else the per-position records of launch_eq_records
void launch_sbool_msg(const uint32_t* keys, const Fr* val, const uint32_t* count, uint32_t upper, const Fr* eq,
                      const Fr* weights, uint32_t vars_left, bool ones, const RoundScratch& sc, cudaStream_t s);
// rec[3 p .. 3 p + 2] for every position p of the 2 * pairs entries of eq: {eq(0), eq(2), 2 eq(3)} (p even) or
// {eq(1), 2 eq(2), 3 eq(3)} (p odd) of p's pair
void launch_eq_records(const Fr* eq, uint64_t pairs, Fr* rec, int sm_count, cudaStream_t s);
void launch_sbool_final(const uint32_t* keys, const Fr* val, const uint32_t* count, const Fr* eq, const Fr* weights,
                        uint32_t n_terms, Fr* out, cudaStream_t s);
void launch_fill_ones(Fr* out, uint32_t n, int sm_count, cudaStream_t s);
void launch_general_msg(const Fr* const* tables_dev, const Fr* scalars, const Fr* eq, uint32_t n_terms, uint32_t n_factors,
                        uint64_t pairs, const RoundScratch& sc, cudaStream_t s);
void launch_general_final(const Fr* const* tables_dev, const Fr* scalars, const Fr* eq, uint32_t n_terms,
                          uint32_t n_factors, Fr* table_vals, Fr* out, cudaStream_t s);

// tail.cu
struct StrobeState;
constexpr uint64_t kReplicateEntries = 1ull << 18;  // sharded proves: gather the tables once all ranks together hold this few entries
constexpr uint32_t kTailMax = 1024;  // entries per table the single-block tail kernel takes over at
// r_dev / st_dev (device pointers, both or neither): take the challenge to bind first and the transcript
// state from device memory (left there by the resident kernel) instead of from r / st.
int launch_tail(int num_poly, const Fr* const* src, uint32_t size, bool fold_first, const Fr& r, const StrobeState& st,
                Fr* out_msgs, Fr* out_chal, Fr* out_final, StrobeState* out_st, cudaStream_t stream,
                const Fr* r_dev = nullptr, const StrobeState* st_dev = nullptr);

// Exchange of round messages between the ranks of a sharded prove through peer memory (comm.cu).
// Every rank owns one ExchangeBox in its own HBM and holds a peer mapping of every other rank's.
// A value crosses as eight 8-byte words {limb, exchange number}: an aligned 8-byte store arrives
// whole, so a word that shows the expected number carries its limb, and neither fences nor a
// separate flag are needed (one NVLink store latency per exchange).  An exchange with number x uses
// slot set x & 1: a rank stores its values into slot [its rank] of every rank's box, then polls its
// own box until every rank's words show x and adds the values in rank order.  Ranks only write
// remotely and read locally; a rank is at most one exchange ahead of the slowest, so two slot sets
// are enough.
constexpr int kPeerRanks = 16;   // ranks a box has slots for (one NVSwitch domain)
constexpr int kPeerVals = 16;    // values per exchange (a round message has at most 5)
constexpr uint32_t kGatherEntries = 1u << 14;  // entries per gathered table: the hand-over of a sharded prove to the rounds every rank runs on its own
struct ExchangeBox {
  uint2 words[2][kPeerRanks][kPeerVals][8];
  // hand-over of a sharded prove to the single-block tail: every rank's chunk of each table, stored
  // here by the ranks themselves (plain stores, a system-wide fence, then the flag)
  Fr gather[kMaxPolys][kGatherEntries];
  unsigned int gather_flag[kPeerRanks];
};
struct PeerTable {
  ExchangeBox* box[kPeerRanks];
};
struct PeerExchange {
  PeerTable peers;
  int rank, world;
  unsigned int xseq_base;   // exchanges made before this launch (the same on every rank)
  unsigned int spin_limit;  // polls (32 ns apart) before a wait gives up
};

// comm.cu: every rank stores its m-entry chunk of each of the L tables at position rank * m of gather[i]
// in every rank's box and waits (bounded) for the other ranks' chunks; *error_word is set when a wait
// ran out.  On success *tables_out[i] points at this rank's complete gather[i].
#ifdef __CUDACC__
// One exchange by a whole block of nthreads threads (all must call): vals[0 .. n_vals) in shared or
// global memory is replaced by the sum over the ranks.  stage: world * n_vals * 8 words of shared
// memory.  Returns false (to every thread) when a wait ran out.
__device__ __forceinline__ bool peer_exchange_sum(const PeerExchange& px, unsigned int xseq, Fr* vals, int n_vals,
                                                  uint32_t* stage, int* ok_shared, int tid, int nthreads) {
  const int par = xseq & 1u;
  const int words = px.world * n_vals * 8;
  if (tid == 0) *ok_shared = 1;
  __syncthreads();
  for (int k = tid; k < words; k += nthreads) {
    const int r = k / (n_vals * 8), rem = k - r * (n_vals * 8), c = rem >> 3, limb = rem & 7;
    uint2* dst = &px.peers.box[r]->words[par][px.rank][c][limb];
    const uint32_t v = vals[c].v[limb];
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(v), "r"(xseq) : "memory");
  }
  const ExchangeBox* mine = px.peers.box[px.rank];
  for (int k = tid; k < words; k += nthreads) {
    const int r = k / (n_vals * 8), rem = k - r * (n_vals * 8), c = rem >> 3, limb = rem & 7;
    const uint2* src = &mine->words[par][r][c][limb];
    uint32_t v, q;
    unsigned int polls = 0;
    for (;;) {
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(q) : "l"(src) : "memory");
      if (q == xseq) break;
      if (++polls > px.spin_limit || *reinterpret_cast<volatile int*>(ok_shared) == 0) {
        *reinterpret_cast<volatile int*>(ok_shared) = 0;
        break;
      }
      __nanosleep(32);
    }
    stage[k] = v;
  }
  __syncthreads();
  const bool ok = *ok_shared != 0;
  if (ok && tid < n_vals) {
    Fr sum = Fr::zero();
    for (int r = 0; r < px.world; r++) {
      Fr v;
#pragma unroll
      for (int i = 0; i < 8; i++) v.v[i] = stage[(r * n_vals + tid) * 8 + i];
      sum = add(sum, v);
    }
    vals[tid] = sum;
  }
  __syncthreads();
  return ok;
}
#endif

// resident.cu
struct ResidentShared;
struct ResidentToEnd {    // launch_resident runs to the end of the protocol
  uint32_t ahead_log;     // tables of at most 2^ahead_log entries: rounds prepared ahead of their challenge
  Fr* out_final;          // L table values at the challenge point, then their product
  StrobeState* out_st;    // transcript state after the last challenge
  uint32_t* ahead_from;   // host: first round that was prepared ahead of its challenge (for diagnostics)
  bool pending;           // the tables still have to be bound on sh->challenge, left with the transcript state in sh->st by
                          // the launch before (which stopped early): log2(size) - 1 messages remain, all prepared ahead;
                          // message k of them goes to out_msgs[(k + 1) * (L + 1)], its challenge to out_chal[k + 1]
};
// px != nullptr: the tables are this rank's chunks of a sharded instance; every round's message is the
// sum over the ranks, exchanged through the peer boxes by the block that completes the local sums.
int launch_resident(int num_poly, const Fr* const* src, Fr* const* ping, Fr* const* pong, uint64_t size, uint32_t rounds,
                    const StrobeState& st, Fr* partials, int max_blocks, int sm_count, ResidentShared* sh, Fr* out_msgs,
                    Fr* out_chal, cudaStream_t stream, const PeerExchange* px = nullptr, const ResidentToEnd* to_end = nullptr);

// sparse.cu
// exchange != nullptr (one rank of a sharded instance, sc.sink publishes to the host): the kernel's last block
// exchanges the message with the other ranks' kernels as exchange number xseq and publishes the sum.
void launch_sparse_msg(uint32_t* idx, Fr* val, const uint32_t* count, uint32_t upper, const Fr* dense,
                       const Fr* pending, const Fr* bind, const RoundScratch& sc, cudaStream_t s,
                       const PeerExchange* exchange = nullptr, unsigned int xseq = 0);
void launch_sparse_bind(uint32_t* idx, Fr* val, const uint32_t* count, uint32_t upper, const Fr& r, int sm_count,
                        cudaStream_t s);
void launch_scatter_runs(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, Fr* dense,
                         int sm_count, cudaStream_t s);
int launch_sparse_fold(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, const Fr& r,
                       uint32_t* block_counts, uint32_t* idx_out, Fr* val_out, uint32_t* count_out, cudaStream_t s);
void launch_scatter(const uint32_t* idx, const Fr* val, const uint32_t* count, uint32_t upper, Fr* dense,
                    int sm_count, cudaStream_t s);
void launch_check_sorted(const uint32_t* idx, uint32_t n, uint64_t limit, uint32_t* bad, int sm_count, cudaStream_t s);
void launch_check_bound(const uint32_t* idx, uint32_t n, uint64_t limit, uint32_t* bad, int sm_count, cudaStream_t s);
void launch_narrow_idx(const uint64_t* in, uint32_t n, uint32_t* out, uint32_t* bad, int sm_count, cudaStream_t s,
                       uint64_t clamp_below = 0);
void launch_sd_final(const uint32_t* idx, const Fr* val, const uint32_t* count, const Fr* dense, Fr* out,
                     cudaStream_t s);

}  // namespace zk
