// The library context and small host helpers shared by the C ABI translation units.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdarg>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "internal.hpp"
#include "merlin.hpp"

namespace zk {

int fail(int code, const char* fmt, ...);

#define ZK_CUDA(call)                                                                        \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) return ::zk::fail(-3 /*ZK_ERR_CUDA*/, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

inline Fr fr_load(const uint64_t* p) {
  Fr x;
  memcpy(x.v, p, 32);
  return x;
}
inline void fr_store(uint64_t* p, const Fr& x) { memcpy(p, x.v, 32); }

// CryptoField::to_bytes_le + Transcript::append_scalar (util/poly.rs:79-83, transcript.rs:27-30):
// the 32-byte canonical little-endian value is absorbed.
inline void transcript_append_scalar(MerlinTranscript& t, const uint8_t* label, size_t n, const Fr& mont) {
  const Fr c = from_mont(mont);
  t.append_message(label, n, reinterpret_cast<const uint8_t*>(c.v), 32);
}
// Transcript::challenge_scalar (transcript.rs:38-42) with CryptoField::from_bytes_le
// (util/poly.rs:72-78): 64 bytes are drawn, the first 32 are reduced mod r.
inline Fr transcript_challenge_scalar(MerlinTranscript& t, const uint8_t* label, size_t n) {
  uint8_t buf[64];
  t.challenge_bytes(label, n, buf, 64);
  Fr raw;
  memcpy(raw.v, buf, 32);
  return to_mont(raw);  // Montgomery product with R^2 also reduces mod r
}

}  // namespace zk

struct MsmStatsPod {
  int window_bits = 0, windows = 0, max_bits = 0;
  uint32_t entries = 0, buckets = 0;
};

struct zk_comm;

constexpr size_t kFinalHostOffset = 7168;  // zk_ctx::host_small: where the final values land when they are read back with the rounds

struct zk_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t side_stream = nullptr;  // a bandwidth-bound pass that may run beside latency-bound launches
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  zk::RoundScratch rs{};
  zk::Fr* final_out = nullptr;   // kMaxPolys + 1 elements
  void* tail_out = nullptr;      // device-resident rounds: messages, challenges, transcript state (8 KiB)
  void* resident_sh = nullptr;   // zk::ResidentShared: hand-over area of the resident multi-round kernel (8 KiB)
  zk::Fr* tail_buf = nullptr;    // sharded proves: gathered values and the last log2(world) rounds' tables
  void* host_small = nullptr;    // pinned, 8 KiB: round messages and other tiny read-backs
  void* mailbox = nullptr;       // pinned + mapped: message kernels publish here, the host polls
  void* work = nullptr;          // grow-only device scratch (copies of caller data, round buffers)
  size_t work_bytes = 0;
  void* aux = nullptr;           // second grow-only scratch (MSM sort and bucket storage)
  size_t aux_bytes = 0;
  void* cmp = nullptr;           // third grow-only scratch (compact small scalars of the MSM)
  size_t cmp_bytes = 0;
  uint64_t replicate_entries = zk::kReplicateEntries;  // sharded proves gather the tables at this many entries in all (0: never)
  bool final_on_host = false;    // the dense round loop read final_out back together with its rounds (host_small + kFinalHostOffset)
  bool sharded_finished = false; // set by the dense round loop of a sharded prove when it gathered the tables and ran to the end
  bool peer_exchange = true;     // sharded proves exchange round messages through peer memory when the ranks could map it
  uint32_t exchange_wait_ms = 16000;  // bound of a device-side wait for another rank's words (ZK_OPT_EXCHANGE_WAIT_MS)
  uint32_t ahead_log = 15;       // dense tables of at most 2^ahead_log entries: rounds prepared ahead of their challenge (ZK_OPT_AHEAD_LOG)
  bool device_tail = true;       // run the last dense rounds in the single-block kernel (zk_set_option turns it off)
  // host clock (microseconds since the first entry) at which each host-stepped round of the most recent
  // proves had its challenge: where the time of a prove goes, round by round (zk_round_times)
  std::vector<double> round_times;
  std::chrono::steady_clock::time_point round_t0;
  void time_mark() {  // one more entry of round_times: now
    if (round_times.size() >= 4096) return;
    const auto now = std::chrono::steady_clock::now();
    if (round_times.empty()) round_t0 = now;
    round_times.push_back(std::chrono::duration<double, std::micro>(now - round_t0).count());
  }
  MsmStatsPod last_msm;          // shape of the most recent MSM (window width, windows, entries)
  uint64_t msm_entries_sum = 0;  // digit entries (= bucket additions) of every MSM since the last zk_msm_work reset
  uint64_t msm_bucket_sum = 0;   // buckets reduced by those MSMs
  uint64_t msm_calls = 0;
  std::atomic<uint64_t> launches{0};
  // Lanes.  The handle a caller holds is the primary lane; calls that arrive while it is busy (the reference opens
  // its commitments from many rayon workers at once, dag/mod.rs:893-905) run on further lanes, each a context of
  // its own (stream, scratch, mailbox) on the same device, created when first needed and kept.  Device objects
  // the caller passes in (SRS handles, device buffers) are shared and only read.
  zk_ctx* primary = nullptr;        // on an extra lane: the handle it belongs to
  std::vector<zk_ctx*> lanes;       // on the primary: the extra lanes
  int max_lanes = 4;                // lanes in all, the primary included (ZK_OPT_LANES)
  bool busy = false;                // guarded by the primary's pool_mu
  std::mutex pool_mu;
  std::condition_variable pool_cv;
  zk_ctx* acquire_lane(bool primary_only);
  void release_lane(zk_ctx* lane);
  uint64_t total_launches() const;

  // Optional per-kernel-kind timing with CUDA events on the context's stream.
  static constexpr int kProfKinds = 8;
  bool prof_on = false;
  struct ProfSpan { cudaEvent_t e0, e1; int kind; };
  std::vector<ProfSpan> prof_spans;
  size_t prof_used = 0;
  uint64_t prof_launches[kProfKinds] = {0};
  double prof_bytes[kProfKinds] = {0};
  double prof_ms[kProfKinds] = {0};
  void prof_begin(int kind, double bytes, int n_launches = 1);
  void prof_end();
  int prof_collect();  // after a stream sync: fold finished spans into prof_ms

  int setup();
  void teardown();
  // Make the scratch at least `bytes` large and return it (contents undefined).
  // Scratch for the next message-producing launch: a fresh sequence number; with `partial`
  // (multi-GPU: the launch yields only this rank's share) the kernel does not publish.
  zk::RoundScratch next_msg_scratch(bool partial) {
    rs.sink.seq++;
    zk::RoundScratch sc = rs;
    if (partial) sc.sink.pub_flag = nullptr;
    return sc;
  }
  int reserve_work(size_t bytes, void** out);
  int reserve_aux(size_t bytes, void** out);
  int reserve_cmp(size_t bytes, void** out);
};

struct zk_transcript {
  zk::MerlinTranscript m;
  zk_transcript(const uint8_t* label, size_t n) : m(label, n) {}
};

namespace zk {
typedef int (*fs_round_fn_t)(void* user, const uint64_t* msgs, uint32_t n_msgs, uint64_t challenge_out[4]);
bool comm_peer_args(const zk_ctx* ctx, const zk_comm* c, PeerExchange* out);
void comm_peer_advance(zk_comm* c, unsigned int n);
int comm_peer_gather(zk_ctx* ctx, zk_comm* c, int n_tables, const Fr* const* chunks, uint32_t m, unsigned int* error_word,
                     const Fr** tables_out);
int fs_round(zk_ctx* ctx, zk_comm* comm, int n_msgs, uint32_t round, fs_round_fn_t fs, void* fs_user, zk_transcript* tr,
             uint64_t* round_msgs, uint64_t* challenges, Fr* challenge,
             bool exchanged_by_kernel = false);
int linear_rounds(zk_ctx* ctx, zk_comm* comm, int L, uint32_t rounds, const Fr** cur, Fr** ping, Fr** pong,
                  uint32_t round_offset, fs_round_fn_t fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                  uint64_t* challenges, Fr* challenge, bool* finals_done);
int check_round_chain(const uint64_t* round_msgs, const uint64_t* challenges, uint32_t rounds, int n_msgs);
int sharded_tail(zk_ctx* ctx, zk_comm* comm, int L, uint32_t n_local, fs_round_fn_t fs, void* fs_user,
                 zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges, Fr* challenge);
// comm.cu
int comm_world(const zk_comm* c);
int exchange_counts(zk_ctx* ctx, zk_comm* comm, uint32_t mine, uint32_t* out);  // api.cu: every rank's count, through the message exchange
int comm_rank(const zk_comm* c);
int comm_sum_fr(zk_ctx* ctx, zk_comm* c, Fr* vals, int n_vals);
int comm_gather_fr(zk_ctx* ctx, zk_comm* c, const Fr* vals, int n_vals, Fr* out);
int comm_gather_bytes(zk_ctx* ctx, zk_comm* c, const void* send, size_t bytes, void* recv);
// A communicator is retired by the first sharded call that fails on it: the ranks' exchange counters may have
// parted (one rank returned early, the others ran on into a wait), and words of the aborted exchange are
// still in the boxes.  Every later sharded call returns ZK_ERR_COMM at once, on every rank that saw a
// failure, until the host frees the communicator and makes a new one on all ranks.
bool comm_poisoned(const zk_comm* c);
void comm_poison(zk_comm* c);
template <class F>
int sharded_call(zk_comm* comm, const char* name, F&& body) {
  if (comm_poisoned(comm))
    return fail(-6 /*ZK_ERR_COMM*/, "%s: an earlier sharded call failed on this communicator; free it and call zk_comm_init again on every rank", name);
  const int rc = body();
  if (rc != 0) comm_poison(comm);
  return rc;
}

// Gives the calling thread a lane of the context for the duration of a call and makes its device current.  Entry
// points go on with `ctx = lk.lane`.  primary_only: the call needs the primary lane itself (sharded calls, whose
// communicator is tied to it, and calls that read or set state kept there); it waits until that lane is free.
struct CtxLock {
  zk_ctx* owner;
  zk_ctx* lane;
  explicit CtxLock(zk_ctx* c, bool primary_only = false) : owner(c->primary ? c->primary : c) {
    lane = owner->acquire_lane(primary_only);
    cudaSetDevice(lane->device);
  }
  ~CtxLock() { owner->release_lane(lane); }
  CtxLock(const CtxLock&) = delete;
  CtxLock& operator=(const CtxLock&) = delete;
};
}  // namespace zk
