// C ABI layer: context, transcript objects and the host-side round loops that drive the
// kernels.  See include/zkb200.h for the contract of every entry point.
#include "../../include/zkb200.h"
#include "ctx.hpp"
#include "strobe_dev.cuh"

#include <chrono>
#include <cstdio>
#include <string>

using namespace zk;

namespace zk {
thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}
}  // namespace zk

namespace zk {
// The kernel that completes a message publishes it to the host-mapped mailbox and then writes this launch's
// sequence number: poll for it instead of synchronising the stream.  `exchanged`: the message went through the
// ranks' exchange, whose kernel reports a wait that ran out in the word beside the sequence word.
int wait_mailbox(zk_ctx* ctx, bool exchanged, uint32_t round) {
  volatile unsigned int* flag =
      reinterpret_cast<volatile unsigned int*>(reinterpret_cast<char*>(ctx->mailbox) + 16 * sizeof(Fr));
  const unsigned int want = ctx->rs.sink.seq;
  const auto t0 = std::chrono::steady_clock::now();
  uint64_t spins = 0;
  while (*flag != want) {
    if ((++spins & 0x3fff) == 0) {
      cudaError_t e = cudaStreamQuery(ctx->stream);
      if (e != cudaSuccess && e != cudaErrorNotReady) return fail(ZK_ERR_CUDA, "round kernel failed: %s", cudaGetErrorString(e));
      const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      if (e == cudaSuccess && *flag != want && waited > 1.0)
        return fail(ZK_ERR_TIMEOUT, "round %u: the stream drained without publishing the message", round);
      if (waited > 60.0) return fail(ZK_ERR_TIMEOUT, "round %u: no message after 60 s", round);
    }
  }
  if (exchanged) {
    volatile unsigned int* err = reinterpret_cast<volatile unsigned int*>(reinterpret_cast<char*>(ctx->mailbox) + 16 * sizeof(Fr) + 4);
    if (*err != 0) {
      *err = 0;  // only the peer-exchange kernel writes the word: leave it clear for rounds that take the NCCL path
      return fail(ZK_ERR_TIMEOUT, "round %u: the other ranks' partial sums did not arrive", round);
    }
  }
  return ZK_OK;
}

// Every rank's 32-bit count in one exchange (the same machinery as a round message: peer stores or an NCCL
// all-gather, published to the polling host): rank r puts its count into a 64-bit slot of its own in one of up
// to four values, so that the sum over the ranks is the list of counts.  out: world counts.
int exchange_counts(zk_ctx* ctx, zk_comm* comm, uint32_t mine, uint32_t* out) {
  const int world = comm_world(comm), rank = comm_rank(comm);
  if (world > 16) return fail(ZK_ERR_ARG, "exchange_counts: more than 16 ranks");
  Fr* enc = reinterpret_cast<Fr*>(ctx->host_small);
  for (int i = 0; i < 4; i++) enc[i] = Fr::zero();
  enc[rank / 4].v[2 * (rank % 4)] = mine;
  (void)ctx->next_msg_scratch(true);  // a sequence number for this exchange
  ZK_CUDA(cudaMemcpyAsync(ctx->rs.sink.msg, enc, 4 * sizeof(Fr), cudaMemcpyHostToDevice, ctx->stream));
  int rc = comm_sum_fr(ctx, comm, ctx->rs.sink.msg, 4);
  if (rc) return rc;
  rc = wait_mailbox(ctx, true, 0);
  if (rc) return rc;
  const Fr* sum = reinterpret_cast<const Fr*>(ctx->mailbox);
  for (int r = 0; r < world; r++) out[r] = sum[r / 4].v[2 * (r % 4)];
  return ZK_OK;
}

// Reads the round message the last kernel left in rs.msg, records it, runs the Fiat-Shamir
// step (callback or built-in transcript) and records the challenge.
int fs_round(zk_ctx* ctx, zk_comm* comm, int n_msgs, uint32_t round, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
             uint64_t* round_msgs, uint64_t* challenges, Fr* challenge, bool exchanged_by_kernel) {
  ZK_CUDA(cudaGetLastError());
  if (comm && !exchanged_by_kernel) {  // every rank holds a partial message: sum them so all ranks absorb the same scalars
    int rc = comm_sum_fr(ctx, comm, ctx->rs.sink.msg, n_msgs);
    if (rc) return rc;
  }
  {
    const int rc = wait_mailbox(ctx, comm != nullptr, round);
    if (rc) return rc;
  }
  const Fr* msg = reinterpret_cast<const Fr*>(ctx->mailbox);
  uint64_t* out_msg = round_msgs + (uint64_t)round * n_msgs * 4;
  for (int c = 0; c < n_msgs; c++) fr_store(out_msg + 4 * c, msg[c]);
  if (fs) {
    uint64_t ch[4];
    if (fs(fs_user, out_msg, (uint32_t)n_msgs, ch) != 0)
      return fail(ZK_ERR_FS_CALLBACK, "Fiat-Shamir callback failed in round %u", round);
    *challenge = fr_load(ch);
  } else {
    for (int c = 0; c < n_msgs; c++) transcript_append_scalar(tr->m, (const uint8_t*)"round_message", 13, msg[c]);
    *challenge = transcript_challenge_scalar(tr->m, (const uint8_t*)"challenge", 9);
  }
  fr_store(challenges + 4 * (uint64_t)round, *challenge);
  ctx->time_mark();
  return ZK_OK;
}
}  // namespace zk

extern "C" {

const char* zk_last_error(void) { return g_last_error.c_str(); }

int zk_init(int device, zk_ctx** out) {
  if (!out) return fail(ZK_ERR_ARG, "zk_init: out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return fail(ZK_ERR_CUDA, "zk_init: no CUDA device: %s", cudaGetErrorString(e));
  if (device < 0 || device >= count) return fail(ZK_ERR_ARG, "zk_init: device %d out of range (%d present)", device, count);
  zk_ctx* c = new zk_ctx();
  c->device = device;
  int rc = c->setup();
  if (rc != ZK_OK) {
    delete c;
    return rc;
  }
  *out = c;
  return ZK_OK;
}

void zk_free(zk_ctx* ctx) {
  if (!ctx) return;
  ctx->teardown();
  delete ctx;
}

uint64_t zk_launch_count(const zk_ctx* ctx) { return ctx ? ctx->total_launches() : 0; }

int zk_set_option(zk_ctx* ctx, int option, int value) {
  if (!ctx) return fail(ZK_ERR_ARG, "zk_set_option: NULL context");
  CtxLock lk(ctx, true);
  std::vector<zk_ctx*> all = ctx->lanes;  // an option holds for every lane of the context
  all.push_back(ctx);
  for (zk_ctx* c : all) {
    switch (option) {
      case ZK_OPT_DEVICE_TAIL: c->device_tail = value != 0; break;
      case ZK_OPT_PEER_EXCHANGE: c->peer_exchange = value != 0; break;
      case ZK_OPT_EXCHANGE_WAIT_MS:
        if (value < 1 || value > 600000) return fail(ZK_ERR_ARG, "zk_set_option: exchange wait out of range (1 .. 600000 ms)");
        c->exchange_wait_ms = (uint32_t)value;
        break;
      case ZK_OPT_REPLICATE_LOG:
        if (value < 0 || value > 30) return fail(ZK_ERR_ARG, "zk_set_option: replicate threshold out of range");
        c->replicate_entries = value == 0 ? 0 : 1ull << value;
        break;
      case ZK_OPT_AHEAD_LOG:
        if (value < 0 || value > 24) return fail(ZK_ERR_ARG, "zk_set_option: run-ahead threshold out of range (0 .. 24)");
        c->ahead_log = (uint32_t)value;
        break;
      case ZK_OPT_LANES:
        if (value < 1 || value > 64) return fail(ZK_ERR_ARG, "zk_set_option: 1 to 64 lanes");
        if (c == ctx) ctx->max_lanes = value;
        break;
      default: return fail(ZK_ERR_ARG, "zk_set_option: unknown option %d", option);
    }
  }
  return ZK_OK;
}

int zk_round_times(zk_ctx* ctx, double* out_us, uint32_t cap, uint32_t* n) {
  if (!ctx || !n) return fail(ZK_ERR_ARG, "zk_round_times: NULL argument");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  *n = (uint32_t)ctx->round_times.size();
  for (uint32_t i = 0; i < *n && i < cap && out_us; i++) out_us[i] = ctx->round_times[i];
  ctx->round_times.clear();
  return ZK_OK;
}

void* zk_stream(zk_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int zk_profile_enable(zk_ctx* ctx, int on) {
  if (!ctx) return fail(ZK_ERR_ARG, "zk_profile_enable: NULL context");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  int rc = ctx->prof_collect();
  if (rc) return rc;
  ctx->prof_on = on != 0;
  if (on) {
    for (int k = 0; k < zk_ctx::kProfKinds; k++) {
      ctx->prof_launches[k] = 0;
      ctx->prof_bytes[k] = 0;
      ctx->prof_ms[k] = 0;
    }
  }
  return ZK_OK;
}

int zk_profile_get(zk_ctx* ctx, int kind, uint64_t* launches, double* ms, double* bytes) {
  if (!ctx || kind < 0 || kind >= zk_ctx::kProfKinds) return fail(ZK_ERR_ARG, "zk_profile_get: bad argument");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  int rc = ctx->prof_collect();
  if (rc) return rc;
  if (launches) *launches = ctx->prof_launches[kind];
  if (ms) *ms = ctx->prof_ms[kind];
  if (bytes) *bytes = ctx->prof_bytes[kind];
  return ZK_OK;
}

int zk_device_alloc(zk_ctx* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return fail(ZK_ERR_ARG, "zk_device_alloc: NULL argument");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaError_t e = cudaMalloc(out, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ZK_ERR_OOM, "zk_device_alloc: %zu bytes: %s", bytes, cudaGetErrorString(e));
  }
  return ZK_OK;
}

int zk_device_free(zk_ctx* ctx, void* ptr) {
  if (!ctx) return fail(ZK_ERR_ARG, "zk_device_free: NULL context");
  CtxLock lk(ctx);
  ctx = lk.lane;
  ZK_CUDA(cudaFree(ptr));
  return ZK_OK;
}

int zk_device_copy(zk_ctx* ctx, void* dst, zk_mem dst_mem, const void* src, zk_mem src_mem, size_t bytes) {
  if (!ctx || (bytes && (!dst || !src))) return fail(ZK_ERR_ARG, "zk_device_copy: NULL argument");
  CtxLock lk(ctx);
  ctx = lk.lane;
  ZK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  (void)dst_mem;
  (void)src_mem;
  return ZK_OK;
}

int zk_device_sync(zk_ctx* ctx) {
  if (!ctx) return fail(ZK_ERR_ARG, "zk_device_sync: NULL context");
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  for (zk_ctx* l : ctx->lanes) ZK_CUDA(cudaStreamSynchronize(l->stream));
  return ZK_OK;
}

// ---------------------------------------------------------------------------- transcript
zk_transcript* zk_transcript_new(const uint8_t* label, size_t label_len) { return new zk_transcript(label, label_len); }
zk_transcript* zk_transcript_clone(const zk_transcript* t) { return t ? new zk_transcript(*t) : nullptr; }
void zk_transcript_free(zk_transcript* t) { delete t; }

void zk_transcript_append_message(zk_transcript* t, const uint8_t* label, size_t label_len, const uint8_t* msg,
                                  size_t msg_len) {
  t->m.append_message(label, label_len, msg, msg_len);
}
void zk_transcript_append_u64(zk_transcript* t, const uint8_t* label, size_t label_len, uint64_t value) {
  t->m.append_u64(label, label_len, value);
}
void zk_transcript_append_scalar(zk_transcript* t, const uint8_t* label, size_t label_len, const uint64_t scalar[4]) {
  transcript_append_scalar(t->m, label, label_len, fr_load(scalar));
}
void zk_transcript_challenge_bytes(zk_transcript* t, const uint8_t* label, size_t label_len, uint8_t* out, size_t n) {
  t->m.challenge_bytes(label, label_len, out, n);
}
void zk_transcript_challenge_scalar(zk_transcript* t, const uint8_t* label, size_t label_len, uint64_t out[4]) {
  fr_store(out, transcript_challenge_scalar(t->m, label, label_len));
}

// ---------------------------------------------------------------------------- linear sumcheck
}  // extern "C"

namespace zk {

// `rounds` rounds of the dense prover over device tables cur[i] of 2^rounds elements each; the
// folded tables alternate between ping and pong.  On return cur[] points at the two-entry
// tables the last challenge has not been bound on yet (or the inputs when rounds == 0), unless
// *finals_done is set: then the single-block tail kernel ran the last rounds with the built-in
// transcript on the device and ctx->final_out already holds the final values.
int linear_rounds(zk_ctx* ctx, zk_comm* comm, int L, uint32_t rounds, const Fr** cur, Fr** ping, Fr** pong,
                  uint32_t round_offset, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                  uint64_t* challenges, Fr* challenge, bool* finals_done) {
  const uint64_t size = 1ull << rounds;
  *finals_done = false;
  ctx->final_on_host = false;
  if (comm) ctx->sharded_finished = false;
  uint64_t cur_size = size;  // entries of the tables cur[] points at
  const bool tail_ok = ctx->device_tail && !fs && tr && !comm;
  uint32_t resident_rounds = 0;  // rounds the resident kernel has produced (their results are still on the device)
  // Reads back what the device-resident rounds left in ctx->tail_out: `left` messages and challenges
  // (rounds round_offset + first ...), the transcript state and the resident kernel's error word.
  // The first `canonical` of them are the multi-round kernel's, which writes canonical integers, not Montgomery form.
  auto collect_device_rounds = [&](uint32_t first, uint32_t left, bool resident, uint32_t canonical) -> int {
    ResidentShared* sh = reinterpret_cast<ResidentShared*>(ctx->resident_sh);
    const size_t bytes = ((size_t)left * (L + 2)) * sizeof(Fr) + sizeof(StrobeState);
    unsigned int* h_flags = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(ctx->host_small) + 8192 - 16);
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->tail_out, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    if (resident) ZK_CUDA(cudaMemcpyAsync(h_flags, sh, 16, cudaMemcpyDeviceToHost, ctx->stream));
    // the final values come back in the same synchronisation (the kernels before this point have written them)
    const bool with_final = bytes <= kFinalHostOffset;  // (always, for tables that fit a GPU)
    if (with_final)
      ZK_CUDA(cudaMemcpyAsync(reinterpret_cast<char*>(ctx->host_small) + kFinalHostOffset, ctx->final_out,
                              (kMaxPolys + 1) * sizeof(Fr), cudaMemcpyDeviceToHost, ctx->stream));
    ZK_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->final_on_host = with_final;
    if (resident && h_flags[2] >= 2) return fail(ZK_ERR_TIMEOUT, "sharded rounds: another rank's partial sums or table chunk did not arrive");
    if (resident && h_flags[2] != 0) return fail(ZK_ERR_TIMEOUT, "resident round kernel: a wait for a challenge ran out");
    Fr* h_msgs = reinterpret_cast<Fr*>(ctx->host_small);
    Fr* h_chal = h_msgs + (size_t)left * (L + 1);
    const StrobeState* h_st = reinterpret_cast<const StrobeState*>(h_chal + left);
    for (uint32_t k = 0; k < left; k++) {
      if (k < canonical) {
        for (int c = 0; c <= L; c++) h_msgs[(size_t)k * (L + 1) + c] = to_mont(h_msgs[(size_t)k * (L + 1) + c]);
        h_chal[k] = to_mont(h_chal[k]);
      }
      for (int c = 0; c <= L; c++)
        fr_store(round_msgs + ((uint64_t)(round_offset + first + k) * (L + 1) + c) * 4, h_msgs[(size_t)k * (L + 1) + c]);
      fr_store(challenges + 4 * (uint64_t)(round_offset + first + k), h_chal[k]);
    }
    *challenge = h_chal[left - 1];
    memcpy(tr->m.strobe().state(), h_st->lanes, 200);
    tr->m.strobe().pos() = (uint8_t)h_st->pos;
    tr->m.strobe().pos_begin() = (uint8_t)h_st->pos_begin;
    tr->m.strobe().cur_flags() = (uint8_t)h_st->cur_flags;
    return ZK_OK;
  };
  auto strobe_now = [&]() {
    StrobeState st;
    memcpy(st.lanes, tr->m.strobe().state(), 200);
    st.pos = tr->m.strobe().pos();
    st.pos_begin = tr->m.strobe().pos_begin();
    st.cur_flags = tr->m.strobe().cur_flags();
    st.pad = 0;
    return st;
  };
  // Sharded prove with the built-in transcript and peer-mapped exchange boxes: the local rounds in one
  // cooperative launch per rank.  Block 0 exchanges a round's local sums with the other ranks' kernels through
  // the boxes (stores over NVLink, bounded wait) and runs the transcript step, so no round returns to the host.
  // The launch stops when the ranks together hold few entries per table; the chunks are gathered (rank order is
  // table order) and every rank finishes on the whole tables by itself, which also covers the rounds of the
  // ranks' own variables.
  PeerExchange px;
  if (comm && ctx->device_tail && !fs && tr && rounds >= 11 && comm_peer_args(ctx, comm, &px) &&
      (uint32_t)px.world <= kTailMax / 2) {
    uint32_t logw = 0;
    while ((1 << logw) < px.world) logw++;
    // The hand-over: when the ranks together hold `gathered_entries` entries per table (last challenge unbound) they
    // store their chunks into each other's boxes and every rank finishes on the whole tables by itself, without
    // further exchanges.  With the multi-block kernel for that (at most three tables) the hand-over is at 2^14
    // entries and the rest runs ahead of its challenges; otherwise at 1024 entries into the single-block kernel.
    const bool own_rest = L <= 3 && ctx->ahead_log >= 2 && rounds + logw >= 15;
    const uint32_t gathered_log = own_rest ? 14 : 10;
    const uint64_t gathered_entries = 1ull << gathered_log;
    const uint32_t R = rounds + 1 + logw - gathered_log;  // messages of the sharded launch
    const uint32_t left = rounds + logw;                   // messages until the end of the protocol
    const size_t bytes = ((size_t)left * (L + 2)) * sizeof(Fr) + sizeof(StrobeState);
    if (R >= 1 && R <= rounds && bytes <= 8192 - 16) {
      const StrobeState st = strobe_now();
      Fr* d_msgs = reinterpret_cast<Fr*>(ctx->tail_out);
      Fr* d_chal = d_msgs + (size_t)left * (L + 1);
      StrobeState* d_st = reinterpret_cast<StrobeState*>(d_chal + left);
      ResidentShared* sh = reinterpret_cast<ResidentShared*>(ctx->resident_sh);
      int rc = ZK_OK;
      ctx->prof_begin(ZK_PROF_ROUND, 64.0 * L * (double)(size / 2) + 192.0 * L * (double)(size / 2));
      const int lrc = launch_resident(L, cur, ping, pong, size, R, st, ctx->rs.sink.partials, ctx->rs.max_blocks,
                                      ctx->sm_count, sh, d_msgs, d_chal, ctx->stream, &px);
      ctx->prof_end();
      if (lrc == 0) {
        ctx->launches++;
        comm_peer_advance(comm, R);
        const Fr* const* last = R == 1 ? cur : (((R - 1) & 1) ? ping : pong);
        const uint64_t m = size >> (R - 1);
        // the ranks store their chunks into each other's boxes (one launch; a wait that runs out lands
        // in the resident kernel's error word, which the read-back below checks)
        const Fr* gathered[kMaxPolys];
        rc = comm_peer_gather(ctx, comm, L, last, (uint32_t)m, &sh->error, gathered);
        if (rc) return rc;
        if (own_rest) {
          Fr* scratch = nullptr;
          rc = ctx->reserve_aux((size_t)L * (gathered_entries / 2 + gathered_entries / 4 + 2) * sizeof(Fr), (void**)&scratch);
          if (rc) return rc;
          Fr *tping[kMaxPolys], *tpong[kMaxPolys];
          for (int i = 0; i < L; i++) {
            tping[i] = scratch + (size_t)i * (gathered_entries / 2);
            tpong[i] = scratch + (size_t)L * (gathered_entries / 2) + (size_t)i * (gathered_entries / 4);
          }
          uint32_t ahead_from = 0;
          // message k of the rest is message R + k of the protocol: the kernel writes it at index k + 1
          const ResidentToEnd te = {ctx->ahead_log, ctx->final_out, d_st, &ahead_from, true};
          if (launch_resident(L, gathered, tping, tpong, gathered_entries, gathered_log, st, ctx->rs.sink.partials,
                              ctx->rs.max_blocks, ctx->sm_count, sh, d_msgs + (size_t)(R - 1) * (L + 1), d_chal + (R - 1),
                              ctx->stream, nullptr, &te))
            return fail(ZK_ERR_CUDA, "sharded rounds: the launch that finishes on the gathered tables failed");
        } else if (launch_tail(L, gathered, kTailMax, true, *challenge, st, d_msgs + (size_t)R * (L + 1), d_chal + R, ctx->final_out,
                               d_st, ctx->stream, &sh->challenge, &sh->st)) {
          return fail(ZK_ERR_CUDA, "tail kernel launch failed");
        }
        ctx->launches++;
        ZK_CUDA(cudaGetLastError());
        rc = collect_device_rounds(0, left, true, own_rest ? left : R);
        if (rc) return rc;
        ctx->sharded_finished = true;
        *finals_done = true;
        return ZK_OK;
      }
      // no cooperative launch on this device: the per-round path below (every rank of one machine takes the same turn)
    }
  }
  for (uint32_t round = 0; round < rounds; round++) {
    if (tail_ok && (cur_size <= kTailMax || round == 0)) {
      // Device-resident rounds: the cooperative multi-block kernel runs the whole protocol (at most three tables);
      // otherwise it runs until kTailMax entries are left and one block finishes in shared memory (at once, for
      // small tables).  Messages, challenges and the transcript state come back in a single copy.
      const StrobeState st = strobe_now();
      const uint32_t left = rounds - round;
      Fr* d_msgs = reinterpret_cast<Fr*>(ctx->tail_out);
      Fr* d_chal = d_msgs + (size_t)left * (L + 1);
      StrobeState* d_st = reinterpret_cast<StrobeState*>(d_chal + left);
      ResidentShared* sh = reinterpret_cast<ResidentShared*>(ctx->resident_sh);
      bool resident = false;
      if (round == 0 && rounds >= 2 && L <= 3 && ctx->ahead_log >= 2 &&
          (size_t)left * (L + 2) * sizeof(Fr) + sizeof(StrobeState) <= 8192 - 16) {
        // All rounds in one cooperative launch: in step while the tables are large, prepared ahead of their
        // challenges once they are small, final values included.
        uint32_t ahead_from = 0;
        const ResidentToEnd te = {ctx->ahead_log, ctx->final_out, d_st, &ahead_from, false};
        ctx->prof_begin(ZK_PROF_ROUND, 64.0 * L * (double)(cur_size / 2) + 192.0 * L * (double)(cur_size / 2));
        const int lrc = launch_resident(L, cur, ping, pong, cur_size, rounds, st, ctx->rs.sink.partials, ctx->rs.max_blocks,
                                        ctx->sm_count, sh, d_msgs, d_chal, ctx->stream, nullptr, &te);
        ctx->prof_end();
        if (lrc == 0) {
          ctx->launches++;
          int rc = collect_device_rounds(0, left, true, left);
          if (rc) return rc;
          *finals_done = true;
          return ZK_OK;
        }
        // no cooperative launch on this device: the kernels below
      }
      if (cur_size > kTailMax) {
        // rounds whose tables (before the fold) are above kTailMax entries: log2(size) - 10 folds + the first
        uint32_t lg = 0;
        while ((1ull << lg) < cur_size) lg++;
        resident_rounds = lg - 9;
        ctx->prof_begin(ZK_PROF_ROUND, 64.0 * L * (double)(cur_size / 2) + 192.0 * L * (double)(cur_size / 2));
        const int lrc = launch_resident(L, cur, ping, pong, cur_size, resident_rounds, st, ctx->rs.sink.partials,
                                        ctx->rs.max_blocks, ctx->sm_count, sh, d_msgs, d_chal, ctx->stream);
        ctx->prof_end();
        if (lrc != 0) {
          resident_rounds = 0;  // no cooperative launch on this device: stay on the per-round kernels
        } else {
          ctx->launches++;
          resident = true;
          Fr** last = ((resident_rounds - 1) & 1) ? ping : pong;
          for (int i = 0; i < L; i++) cur[i] = last[i];
          cur_size >>= (resident_rounds - 1);
        }
      }
      if (cur_size <= kTailMax) {
        const bool fold_first = resident || round > 0;
        if (launch_tail(L, cur, (uint32_t)cur_size, fold_first, *challenge, st, d_msgs + (size_t)resident_rounds * (L + 1),
                        d_chal + resident_rounds, ctx->final_out, d_st, ctx->stream, resident ? &sh->challenge : nullptr,
                        resident ? &sh->st : nullptr))
          return fail(ZK_ERR_CUDA, "tail kernel launch failed");
        ctx->launches++;
        ZK_CUDA(cudaGetLastError());
        int rc = collect_device_rounds(round, left, resident, resident ? resident_rounds : 0);
        if (rc) return rc;
        *finals_done = true;
        return ZK_OK;
      }
    }
    if (comm) {
      // Sharded prove, small tables: a round is then all exchange and no work.  Bind the pending
      // challenge, gather every rank's chunk (the chunks are the table's top index bits, so rank order
      // is table order) and let every rank run the rest of the protocol on the whole table, where the
      // rounds stay on the device.  Every rank computes the same messages, so the transcripts agree.
      const uint64_t after_fold = round == 0 ? cur_size : cur_size >> 1;
      const int world = comm_world(comm);
      if (after_fold * (uint64_t)world <= ctx->replicate_entries && after_fold >= 1) {
        uint32_t logw = 0;
        while ((1 << logw) < world) logw++;
        const uint64_t full = after_fold * world;
        Fr* rep = nullptr;
        int rc = ctx->reserve_aux(((size_t)L * (full + full / 2 + full / 4) + 16) * sizeof(Fr), (void**)&rep);
        if (rc) return rc;
        const Fr* rcur[kMaxPolys];
        Fr *rping[kMaxPolys], *rpong[kMaxPolys];
        for (int i = 0; i < L; i++) {
          const Fr* chunk = cur[i];
          if (round > 0) {
            Fr* dst = ((round & 1) ? ping : pong)[i];
            launch_fold(cur[i], dst, *challenge, after_fold, ctx->rs.max_blocks, ctx->stream);
            ctx->launches++;
            chunk = dst;
          }
          Fr* whole = rep + (size_t)i * full;
          rc = comm_gather_bytes(ctx, comm, chunk, after_fold * sizeof(Fr), whole);
          if (rc) return rc;
          rcur[i] = whole;
          rping[i] = rep + (size_t)L * full + (size_t)i * (full / 2);
          rpong[i] = rep + (size_t)L * (full + full / 2) + (size_t)i * (full / 4);
        }
        uint32_t lg = 0;
        while ((1ull << lg) < full) lg++;
        bool done = false;
        rc = linear_rounds(ctx, nullptr, L, lg, rcur, rping, rpong, round_offset + round, fs, fs_user, tr, round_msgs, challenges,
                           challenge, &done);
        if (rc) return rc;
        if (!done) {
          launch_final(L, lg > 0, rcur, *challenge, ctx->final_out, ctx->stream);
          ctx->launches++;
        }
        ctx->sharded_finished = true;
        *finals_done = true;
        return ZK_OK;
      }
    }
    const uint64_t pairs = size >> (round + 1);
    const RoundScratch sc = ctx->next_msg_scratch(comm != nullptr);
    if (round == 0) {
      ctx->prof_begin(ZK_PROF_ROUND, 64.0 * L * pairs);
      launch_round(L, false, cur, nullptr, *challenge, pairs, sc, ctx->stream);
    } else {
      Fr** dst = (round & 1) ? ping : pong;
      ctx->prof_begin(ZK_PROF_ROUND, 192.0 * L * pairs);
      launch_round(L, true, cur, dst, *challenge, pairs, sc, ctx->stream);
      for (int i = 0; i < L; i++) cur[i] = dst[i];
      cur_size >>= 1;
    }
    ctx->prof_end();
    ctx->launches++;
    int rc = fs_round(ctx, comm, L + 1, round_offset + round, fs, fs_user, tr, round_msgs, challenges, challenge);
    if (rc != ZK_OK) return rc;
  }
  return ZK_OK;
}

// Self-check of a sharded prove on the host, a few microseconds: every summed message must continue the
// round before it, s_m(0) + s_m(1) = s_{m-1}(r_{m-1}) (the identity SumcheckVerifier checks, verifier.rs:
// 7-70).  A share that was damaged on its way between the ranks breaks it on every rank alike, so all
// ranks report ZK_ERR_COMM instead of returning a proof no verifier accepts.  n_msgs = degree + 1 values
// per round at the points 0..degree; Lagrange form with the denominators cleared:
//   degree! * s(r) = sum_i (-1)^(degree-i) C(degree, i) s(i) prod_{j != i} (r - j).
int check_round_chain(const uint64_t* round_msgs, const uint64_t* challenges, uint32_t rounds, int n_msgs) {
  const int d = n_msgs - 1;
  if (d < 1 || d > 8) return ZK_OK;
  uint32_t fact = 1, binom[9];
  for (int i = 1; i <= d; i++) fact *= i;
  binom[0] = 1;
  for (int i = 1; i <= d; i++) binom[i] = binom[i - 1] * (d - i + 1) / i;
  const Fr fact_m = from_u32<FrParams>(fact);
  for (uint32_t m = 1; m < rounds; m++) {
    const uint64_t* prev = round_msgs + (uint64_t)(m - 1) * n_msgs * 4;
    const uint64_t* cur = round_msgs + (uint64_t)m * n_msgs * 4;
    const Fr r = fr_load(challenges + 4 * (uint64_t)(m - 1));
    Fr diff[9];
    for (int j = 0; j <= d; j++) diff[j] = sub(r, from_u32<FrParams>((uint32_t)j));
    Fr rhs = Fr::zero();
    for (int i = 0; i <= d; i++) {
      Fr term = mul(fr_load(prev + 4 * i), from_u32<FrParams>(binom[i]));
      for (int j = 0; j <= d; j++)
        if (j != i) term = mul(term, diff[j]);
      rhs = ((d - i) & 1) ? sub(rhs, term) : add(rhs, term);
    }
    const Fr lhs = mul(fact_m, add(fr_load(cur), fr_load(cur + 4)));
    if (lhs != rhs)
      return fail(ZK_ERR_COMM, "round %u: the summed message does not continue round %u (a rank's share was damaged in the exchange)", m, m - 1);
  }
  return ZK_OK;
}

// After the local rounds of a sharded prove: ctx->final_out[0..L) holds this rank's fully bound
// value of each table.  Gathers them into L tables of `world` entries, runs the remaining
// log2(world) rounds identically on every rank and leaves the final values in ctx->final_out.
int sharded_tail(zk_ctx* ctx, zk_comm* comm, int L, uint32_t n_local, zk_fs_round_fn fs, void* fs_user,
                 zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges, Fr* challenge) {
  const int world = comm_world(comm);
  uint32_t logw = 0;
  while ((1 << logw) < world) logw++;
  Fr* buf = ctx->tail_buf;  // [gathered: world * L][tables: L * world][ping: L * world / 2][pong: L * world / 4]
  Fr* gathered = buf;
  Fr* tables = buf + (size_t)world * kMaxPolys;
  int rc = comm_gather_fr(ctx, comm, ctx->final_out, L, gathered);
  if (rc) return rc;
  // transpose rank-major values into per-table arrays (tiny: through the host)
  Fr host[64 * kMaxPolys], arranged[64 * kMaxPolys];
  ZK_CUDA(cudaMemcpyAsync(host, gathered, (size_t)world * L * sizeof(Fr), cudaMemcpyDeviceToHost, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  for (int r = 0; r < world; r++)
    for (int i = 0; i < L; i++) arranged[i * world + r] = host[r * L + i];
  ZK_CUDA(cudaMemcpyAsync(tables, arranged, (size_t)world * L * sizeof(Fr), cudaMemcpyHostToDevice, ctx->stream));
  const Fr* cur[kMaxPolys];
  Fr *ping[kMaxPolys], *pong[kMaxPolys];
  Fr* pp = tables + (size_t)world * kMaxPolys;
  for (int i = 0; i < L; i++) {
    cur[i] = tables + (size_t)i * world;
    ping[i] = pp + (size_t)i * world;
    pong[i] = pp + (size_t)(kMaxPolys + i) * world;
  }
  bool done = false;
  rc = linear_rounds(ctx, nullptr, L, logw, cur, ping, pong, n_local, fs, fs_user, tr, round_msgs, challenges, challenge, &done);
  if (rc) return rc;
  if (!done) {
    launch_final(L, logw > 0, cur, *challenge, ctx->final_out, ctx->stream);
    ctx->launches++;
  }
  return ZK_OK;
}

int linear_prove_impl(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t num_poly, const uint64_t* const* tables,
                      zk_mem tables_mem, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                      uint64_t* challenges, uint64_t* final_table0, uint64_t* final_eval) {
  if (!ctx) return fail(ZK_ERR_ARG, "linear_prove: NULL context");
  if (!tables || num_poly == 0) return fail(ZK_ERR_ARG, "Polynomials cannot be empty");
  if (num_poly > kMaxPolys) return fail(ZK_ERR_ARG, "linear_prove: num_poly %u exceeds %d", num_poly, kMaxPolys);
  if (num_var > 40) return fail(ZK_ERR_ARG, "linear_prove: num_var %u too large", num_var);
  if (!fs && !tr) return fail(ZK_ERR_ARG, "linear_prove: neither a callback nor a transcript was given");
  for (uint32_t i = 0; i < num_poly; i++)
    if (!tables[i]) return fail(ZK_ERR_ARG, "Polynomial %u has incorrect size", i);
  if (num_var && (!round_msgs || !challenges)) return fail(ZK_ERR_ARG, "linear_prove: NULL output");
  if (!final_eval) return fail(ZK_ERR_ARG, "linear_prove: NULL output");
  const int world = comm_world(comm);
  uint32_t logw = 0;
  while ((1 << logw) < world) logw++;
  if (num_var < logw) return fail(ZK_ERR_ARG, "linear_prove: %u variables cannot be sharded over %d ranks", num_var, world);
  if (world > 64) return fail(ZK_ERR_ARG, "linear_prove: at most 64 ranks");

  CtxLock lk(ctx, world > 1);  // a sharded prove runs on the lane its communicator was made on
  ctx = lk.lane;
  const uint32_t n_local = num_var - logw;
  const uint64_t size = 1ull << n_local;
  const int L = (int)num_poly;

  // device layout: [copies of host inputs] [ping: L * size/2] [pong: L * size/4]
  const uint64_t in_elems = tables_mem == ZK_MEM_HOST ? size * L : 0;
  const uint64_t ping_elems = (size / 2) * L, pong_elems = (size / 4) * L;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((in_elems + ping_elems + pong_elems + 1) * sizeof(Fr), (void**)&base);
  if (rc != ZK_OK) return rc;
  const Fr* cur[kMaxPolys];
  Fr *ping[kMaxPolys], *pong[kMaxPolys];
  for (int i = 0; i < L; i++) {
    if (tables_mem == ZK_MEM_HOST) {
      Fr* d = base + (uint64_t)i * size;
      ZK_CUDA(cudaMemcpyAsync(d, tables[i], size * sizeof(Fr), cudaMemcpyHostToDevice, ctx->stream));
      cur[i] = d;
    } else {
      cur[i] = reinterpret_cast<const Fr*>(tables[i]);
    }
    ping[i] = base + in_elems + (uint64_t)i * (size / 2);
    pong[i] = base + in_elems + ping_elems + (uint64_t)i * (size / 4);
  }

  Fr challenge = Fr::zero();
  bool done = false;
  rc = linear_rounds(ctx, world > 1 ? comm : nullptr, L, n_local, cur, ping, pong, 0, fs, fs_user, tr, round_msgs,
                     challenges, &challenge, &done);
  if (rc) return rc;
  if (!done) {
    launch_final(L, n_local > 0, cur, challenge, ctx->final_out, ctx->stream);
    ctx->launches++;
  }
  if (world > 1 && !ctx->sharded_finished) {
    rc = sharded_tail(ctx, comm, L, n_local, fs, fs_user, tr, round_msgs, challenges, &challenge);
    if (rc) return rc;
  }
  ZK_CUDA(cudaGetLastError());
  const Fr* fin = reinterpret_cast<const Fr*>(reinterpret_cast<char*>(ctx->host_small) + kFinalHostOffset);
  if (!(done && ctx->final_on_host && (world == 1 || ctx->sharded_finished))) {  // not read back with the rounds
    fin = reinterpret_cast<const Fr*>(ctx->host_small);
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->final_out, (L + 1) * sizeof(Fr), cudaMemcpyDeviceToHost, ctx->stream));
    ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  if (final_table0)
    for (int i = 0; i < L; i++) fr_store(final_table0 + 4 * i, fin[i]);
  fr_store(final_eval, fin[L]);
  if (world > 1) return check_round_chain(round_msgs, challenges, num_var, L + 1);
  return ZK_OK;
}

}  // namespace zk

extern "C" {

int zk_sumcheck_linear_prove(zk_ctx* ctx, uint32_t num_var, uint32_t num_poly, const uint64_t* const* tables,
                             zk_mem tables_mem, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
                             uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_table0,
                             uint64_t* final_eval) {
  return linear_prove_impl(ctx, nullptr, num_var, num_poly, tables, tables_mem, fs, fs_user, tr, round_msgs, challenges,
                           final_table0, final_eval);
}

int zk_sumcheck_linear_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t num_poly,
                                     const uint64_t* const* local_tables, zk_mem tables_mem, zk_fs_round_fn fs,
                                     void* fs_user, zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                                     uint64_t* final_table0, uint64_t* final_eval) {
  if (!comm) return fail(ZK_ERR_ARG, "linear_prove_sharded: NULL communicator");
  return sharded_call(comm, "linear_prove_sharded", [&] {
    return linear_prove_impl(ctx, comm, num_var, num_poly, local_tables, tables_mem, fs, fs_user, tr, round_msgs, challenges,
                             final_table0, final_eval);
  });
}

// ---------------------------------------------------------------------------- folds
int zk_fold_lsb(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k, const uint64_t* point,
                uint64_t* out, zk_mem out_mem) {
  if (!ctx || !evals || !out || (k && !point)) return fail(ZK_ERR_ARG, "fold_lsb: NULL argument");
  if (k > n) return fail(ZK_ERR_ARG, "invalid size of partial point");
  if (n > 40) return fail(ZK_ERR_ARG, "fold_lsb: n %u too large", n);
  CtxLock lk(ctx);
  ctx = lk.lane;
  const uint64_t size = 1ull << n;
  const uint64_t in_elems = evals_mem == ZK_MEM_HOST ? size : 0;
  Fr* base = nullptr;
  int rc = ctx->reserve_work((in_elems + size / 2 + size / 4 + 2) * sizeof(Fr), (void**)&base);
  if (rc != ZK_OK) return rc;
  const Fr* cur = reinterpret_cast<const Fr*>(evals);
  if (evals_mem == ZK_MEM_HOST) {
    ZK_CUDA(cudaMemcpyAsync(base, evals, size * sizeof(Fr), cudaMemcpyHostToDevice, ctx->stream));
    cur = base;
  }
  Fr* bufs[2] = {base + in_elems, base + in_elems + size / 2 + 1};
  for (uint32_t i = 0; i < k; i++) {
    Fr* dst = bufs[i & 1];
    ctx->prof_begin(ZK_PROF_FOLD, 96.0 * (double)(size >> (i + 1)));
    launch_fold(cur, dst, fr_load(point + 4 * (uint64_t)i), size >> (i + 1), ctx->rs.max_blocks, ctx->stream);
    ctx->prof_end();
    ctx->launches++;
    cur = dst;
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(out, cur, (size >> k) * sizeof(Fr), cudaMemcpyDefault, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  (void)out_mem;
  return ZK_OK;
}

}  // extern "C"
