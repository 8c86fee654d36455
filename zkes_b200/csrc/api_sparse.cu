// C ABI: sparse x dense product sumcheck (host round loop over the kernels of sparse.cu).
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace {
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Bump allocator over the context's scratch.
struct Arena {
  char* base;
  size_t off = 0;
  template <class T>
  T* take(size_t n) {
    T* p = reinterpret_cast<T*>(base + off);
    off = align_up(off + n * sizeof(T), 256);
    return p;
  }
};
}  // namespace

static int sparse_dense_impl(zk_ctx* ctx, zk_comm* comm, uint32_t total_var, uint64_t nnz, const uint64_t* idx,
                             const uint64_t* vals, const uint64_t* dense, zk_mem mem, zk_fs_round_fn fs, void* fs_user,
                             zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_table0,
                             uint64_t* final_eval) {
  if (!ctx) return fail(ZK_ERR_ARG, "sparse_dense_prove: NULL context");
  const int world = comm_world(comm);
  uint32_t logw = 0;
  while ((1 << logw) < world) logw++;
  if (total_var < logw) return fail(ZK_ERR_ARG, "sparse_dense_prove: %u variables cannot be sharded over %d ranks", total_var, world);
  if (world > 64) return fail(ZK_ERR_ARG, "sparse_dense_prove: at most 64 ranks");
  const uint32_t num_var = total_var - logw;  // variables of this rank's chunk
  if (world == 1) comm = nullptr;
  if (num_var > 32) return fail(ZK_ERR_ARG, "sparse_dense_prove: num_var %u exceeds 32", num_var);
  const uint64_t size = 1ull << num_var;
  if (nnz > size) return fail(ZK_ERR_ARG, "sparse_dense_prove: %llu entries in a domain of %llu", (unsigned long long)nnz, (unsigned long long)size);
  if (!dense || (nnz && (!idx || !vals))) return fail(ZK_ERR_ARG, "sparse_dense_prove: NULL input");
  if (!fs && !tr) return fail(ZK_ERR_ARG, "sparse_dense_prove: neither a callback nor a transcript was given");
  if (!final_eval || (total_var && (!round_msgs || !challenges))) return fail(ZK_ERR_ARG, "sparse_dense_prove: NULL output");

  CtxLock lk(ctx, comm != nullptr);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint32_t K = (uint32_t)nnz;
  // Sharded: every rank must leave the entry form at the same round (the dense rounds exchange
  // differently, and may gather the tables), so the rule below uses the largest entry count of any rank.
  ctx->time_mark();  // call entry
  uint32_t K_rule = K;
  if (comm) {
    uint32_t all[16];
    const int grc = exchange_counts(ctx, comm, K, all);
    if (grc) return grc;
    for (int r = 0; r < world; r++)
      if (all[r] > K_rule) K_rule = all[r];
  }
  // The dense phase starts at the first round whose table size is <= 2 * (entry bound).
  uint64_t dense_cap = 2;
  while (dense_cap < 2 * (uint64_t)K_rule && dense_cap < size) dense_cap <<= 1;

  size_t need = 4096;
  const bool host_in = mem == ZK_MEM_HOST;
  if (host_in) need += align_up(size * sizeof(Fr), 256) + align_up(K * 8ull, 256);
  need += align_up((size / 2 + 1) * sizeof(Fr), 256) + align_up((size / 4 + 1) * sizeof(Fr), 256);
  need += 2 * (align_up((K + 1) * 4ull, 256) + align_up((K + 1) * sizeof(Fr), 256));
  need += align_up((K / 256 + 2) * 4ull, 256) + 1024;
  need += 3 * align_up((dense_cap + 1) * sizeof(Fr), 256) + 2 * align_up((dense_cap / 4 + 1) * sizeof(Fr), 256);
  Arena ar;
  int rc = ctx->reserve_work(need, (void**)&ar.base);
  if (rc != ZK_OK) return rc;

  const Fr* b_cur = reinterpret_cast<const Fr*>(dense);
  const uint64_t* idx64 = idx;
  const Fr* val_in = reinterpret_cast<const Fr*>(vals);
  if (host_in) {
    Fr* d = ar.take<Fr>(size);
    ZK_CUDA(cudaMemcpyAsync(d, dense, size * sizeof(Fr), cudaMemcpyHostToDevice, s));
    b_cur = d;
    uint64_t* di = ar.take<uint64_t>(K + 1);
    if (K) ZK_CUDA(cudaMemcpyAsync(di, idx, K * 8ull, cudaMemcpyHostToDevice, s));
    idx64 = di;
  }
  Fr* b_buf[2] = {ar.take<Fr>(size / 2 + 1), ar.take<Fr>(size / 4 + 1)};
  uint32_t* e_idx[2] = {ar.take<uint32_t>(K + 1), ar.take<uint32_t>(K + 1)};
  Fr* e_val[2] = {ar.take<Fr>(K + 1), ar.take<Fr>(K + 1)};
  uint32_t* block_counts = ar.take<uint32_t>(K / 256 + 2);
  uint32_t* counts = ar.take<uint32_t>(64);  // [0], [1]: entry counts (ping-pong); [2]: bad-input flag
  Fr* a_dense = ar.take<Fr>(dense_cap + 1);
  Fr* d_ping[2] = {ar.take<Fr>(dense_cap / 2 + 1), ar.take<Fr>(dense_cap / 2 + 1)};
  Fr* d_pong[2] = {ar.take<Fr>(dense_cap / 4 + 1), ar.take<Fr>(dense_cap / 4 + 1)};

  // entries: narrow the indices, copy the values, check order
  ZK_CUDA(cudaMemsetAsync(counts, 0, 64 * 4, s));
  ZK_CUDA(cudaMemcpyAsync(counts, &K, 4, cudaMemcpyHostToDevice, s));
  // The order and range of the indices are checked on the device; the host reads the flag when it next hears from
  // the stream (the first round's message), not before: out-of-range indices are clamped, so the kernels in
  // between stay inside their tables whatever the caller passed.
  uint32_t* h_bad = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(ctx->host_small) + 3072);
  bool bad_checked = K == 0;
  if (K) {
    launch_narrow_idx(idx64, K, e_idx[0], counts + 2, ctx->sm_count, s, size);
    launch_check_sorted(e_idx[0], K, size, counts + 2, ctx->sm_count, s);
    ctx->launches += 2;
    ZK_CUDA(cudaMemcpyAsync(e_val[0], val_in, K * sizeof(Fr), cudaMemcpyDefault, s));
    ZK_CUDA(cudaMemcpyAsync(h_bad, counts + 2, 4, cudaMemcpyDeviceToHost, s));
  }
  auto check_bad = [&](bool synchronise) -> int {  // after the stream has passed the copy above
    if (bad_checked) return ZK_OK;
    if (synchronise) ZK_CUDA(cudaStreamSynchronize(s));
    bad_checked = true;
    if (*h_bad) return fail(ZK_ERR_ARG, "sparse_dense_prove: indices must be strictly increasing and below 2^num_var");
    return ZK_OK;
  };

  bool pending = false;  // the dense table still has to be folded by pend_r (done together with the next fold)
  Fr pend_r = Fr::zero();
  auto other_buf = [&](const Fr* cur) { return cur == b_buf[0] ? b_buf[1] : b_buf[0]; };
  const int e = 0;       // the entries are updated in place
  bool e_pending = false;  // the entries still have to be bound on e_r (the next message kernel does it)
  Fr e_r = Fr::zero();
  uint32_t k_upper = K;  // bound on the live entry count
  Fr challenge = Fr::zero();
  uint64_t S = size;
  bool finished = false;  // the dense phase ran to the end (final values are in ctx->final_out)
  bool dense_done = false;  // ... inside the device-resident rounds, which read the final values back with the rounds
  for (uint32_t round = 0; round < num_var; round++, S >>= 1) {
    if (K_rule && S <= dense_cap) {
      // hand over to the dense prover: scatter the entries into a table and run the remaining rounds
      rc = check_bad(true);  // (no entry-form round ran: the flag has not been looked at yet)
      if (rc != ZK_OK) return rc;
      if (pending) {  // not reached with the pairing rule below; kept so the hand-over never sees a stale table
        Fr* nb = other_buf(b_cur);
        launch_fold(b_cur, nb, pend_r, S, ctx->rs.max_blocks, s);
        ctx->launches++;
        b_cur = nb;
        pending = false;
      }
      if (e_pending) {  // the entries still carry the last challenge
        launch_sparse_bind(e_idx[e], e_val[e], counts + e, k_upper, e_r, ctx->sm_count, s);
        ctx->launches++;
        e_pending = false;
      }
      ZK_CUDA(cudaMemsetAsync(a_dense, 0, S * sizeof(Fr), s));
      launch_scatter_runs(e_idx[e], e_val[e], counts + e, k_upper, a_dense, ctx->sm_count, s);
      ctx->launches++;
      const Fr* d_cur[2] = {a_dense, b_cur};
      bool done = false;
      rc = linear_rounds(ctx, comm, 2, num_var - round, d_cur, d_ping, d_pong, round, fs, fs_user, tr, round_msgs,
                         challenges, &challenge, &done);
      if (rc) return rc;
      dense_done = done;
      ctx->time_mark();  // the dense rounds are back
      if (!done) {
        launch_final(2, true, d_cur, challenge, ctx->final_out, s);
        ctx->launches++;
      }
      finished = true;
      break;
    }
    // Sharded over peer memory: the message kernel's last block exchanges the message itself (no launch between)
    PeerExchange px;
    const bool fused = comm && world <= kPeerRanks && ctx->rs.sink.pub_flag && comm_peer_args(ctx, comm, &px);
    const RoundScratch sc = ctx->next_msg_scratch(comm != nullptr && !fused);
    // per live entry: index + value read, one 64-byte pair of b gathered
    ctx->prof_begin(ZK_PROF_SPARSE_MSG, (e_pending ? 144.0 : 104.0) * k_upper);
    launch_sparse_msg(e_idx[e], e_val[e], counts + e, k_upper, b_cur, pending ? &pend_r : nullptr, e_pending ? &e_r : nullptr, sc, s,
                      fused ? &px : nullptr, fused ? px.xseq_base + 1 : 0);
    ctx->prof_end();
    ctx->launches++;
    if (fused) comm_peer_advance(comm, 1);
    rc = fs_round(ctx, comm, 3, round, fs, fs_user, tr, round_msgs, challenges, &challenge, fused);
    if (rc != ZK_OK) return rc;
    rc = check_bad(false);  // the message kernel ran after the copy of the flag
    if (rc != ZK_OK) return rc;
    // Fold of the dense table.  When the next round is still in entry form its message can fold
    // the few values it needs on the fly, so this fold waits and is done together with the next
    // one in a single pass over the table (k_fold2).
    const bool next_sparse = round + 1 < num_var && (!K_rule || (S / 2) > dense_cap);
    // The table fold (bandwidth-bound, long) and the entry fold (three short launches) touch disjoint
    // buffers: the table fold goes to the side stream and the two run side by side.  With the
    // per-kernel profiler on they stay in line so that each span times one kernel alone.
    const bool fold_now = pending || !next_sparse;
    const bool beside = fold_now && !ctx->prof_on;
    cudaStream_t fs_stream = beside ? ctx->side_stream : s;
    if (beside) {
      ZK_CUDA(cudaEventRecord(ctx->ev_fork, s));
      ZK_CUDA(cudaStreamWaitEvent(fs_stream, ctx->ev_fork, 0));
    }
    if (pending) {
      Fr* nb = other_buf(b_cur);
      ctx->prof_begin(ZK_PROF_FOLD, 32.0 * (double)(2 * S + S / 2));
      launch_fold2(b_cur, nb, pend_r, challenge, S / 2, ctx->rs.max_blocks, fs_stream);
      ctx->prof_end();
      ctx->launches++;
      b_cur = nb;
      pending = false;
    } else if (next_sparse) {
      pending = true;
      pend_r = challenge;
    } else {
      Fr* nb = other_buf(b_cur);
      ctx->prof_begin(ZK_PROF_FOLD, 96.0 * (double)(S / 2));
      launch_fold(b_cur, nb, challenge, S / 2, ctx->rs.max_blocks, fs_stream);
      ctx->prof_end();
      ctx->launches++;
      b_cur = nb;
    }
    if (beside) ZK_CUDA(cudaEventRecord(ctx->ev_join, fs_stream));
    // the entries are bound on this challenge by the next message kernel (or at the hand-over), in place
    e_pending = true;
    e_r = challenge;
    if (beside) ZK_CUDA(cudaStreamWaitEvent(s, ctx->ev_join, 0));
  }
  rc = check_bad(true);
  if (rc != ZK_OK) return rc;
  if (!finished && e_pending) {  // the entry form ran to the end (no entries anywhere): bind the last challenge
    launch_sparse_bind(e_idx[e], e_val[e], counts + e, k_upper, e_r, ctx->sm_count, s);
    ctx->launches++;
  }
  if (!finished) {  // no entries, or no variables: the entry form ran to the end
    launch_sd_final(e_idx[e], e_val[e], counts + e, b_cur, ctx->final_out, s);
    ctx->launches++;
  }
  if (comm && !(finished && ctx->sharded_finished)) {  // the remaining log2(world) variables: every rank finishes on the gathered values
    rc = sharded_tail(ctx, comm, 2, num_var, fs, fs_user, tr, round_msgs, challenges, &challenge);
    if (rc) return rc;
  }
  ZK_CUDA(cudaGetLastError());
  const Fr* fin = reinterpret_cast<const Fr*>(reinterpret_cast<char*>(ctx->host_small) + kFinalHostOffset);
  if (!(dense_done && ctx->final_on_host && (!comm || ctx->sharded_finished))) {  // not read back with the dense rounds
    fin = reinterpret_cast<const Fr*>(ctx->host_small);
    ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->final_out, 3 * sizeof(Fr), cudaMemcpyDeviceToHost, s));
    ZK_CUDA(cudaStreamSynchronize(s));
  }
  if (final_table0) {
    fr_store(final_table0, fin[0]);
    fr_store(final_table0 + 4, fin[1]);
  }
  fr_store(final_eval, fin[2]);
  ctx->time_mark();  // call exit
  if (comm) return check_round_chain(round_msgs, challenges, total_var, 3);
  return ZK_OK;
}

extern "C" int zk_sumcheck_sparse_dense_prove(zk_ctx* ctx, uint32_t num_var, uint64_t nnz, const uint64_t* idx,
                                              const uint64_t* vals, const uint64_t* dense, zk_mem mem,
                                              zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
                                              uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_table0,
                                              uint64_t* final_eval) {
  return sparse_dense_impl(ctx, nullptr, num_var, nnz, idx, vals, dense, mem, fs, fs_user, tr, round_msgs, challenges,
                           final_table0, final_eval);
}

extern "C" int zk_sumcheck_sparse_dense_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint64_t local_nnz,
                                                      const uint64_t* local_idx, const uint64_t* local_vals,
                                                      const uint64_t* local_dense, zk_mem mem, zk_fs_round_fn fs,
                                                      void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                                                      uint64_t* challenges, uint64_t* final_table0,
                                                      uint64_t* final_eval) {
  if (!comm) return fail(ZK_ERR_ARG, "sparse_dense_prove_sharded: NULL communicator");
  return sharded_call(comm, "sparse_dense_prove_sharded", [&] {
    return sparse_dense_impl(ctx, comm, num_var, local_nnz, local_idx, local_vals, local_dense, mem, fs, fs_user, tr,
                             round_msgs, challenges, final_table0, final_eval);
  });
}
