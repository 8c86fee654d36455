// C ABI: SparseBoolSumcheckProver and GeneralLinearSumcheckProver (host round loops).
#include "../../include/zkb200.h"
#include "ctx.hpp"

#include <algorithm>
#include <vector>

using namespace zk;

namespace zk {
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table);
size_t keyset_scratch_bytes(uint32_t n_terms, uint32_t num_var);
int keyset_order(zk_ctx* ctx, const uint64_t* positions_dev, const uint64_t* term_begin_dev, uint32_t n_terms, uint64_t total,
                 uint32_t num_var, void* scratch, uint32_t* keys_out, uint32_t bad_host[2]);
int comm_sum_fr_vec(zk_ctx* ctx, zk_comm* c, Fr* vals, uint64_t n);
}

namespace {
inline size_t al(size_t x) { return (x + 255) & ~(size_t)255; }
}

namespace {

// The boolean-check prover; with a communicator the terms given are this rank's share of them (the sum over
// terms is the only thing the ranks have in common: the partial messages and the partial final value are summed
// across the ranks, everything else is local).
int sbool_prove(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t n_terms, const uint64_t* weights,
                const uint64_t* positions, const uint64_t* n_positions, const uint64_t* eq_point,
                zk_fs_round_fn fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                uint64_t* challenges, uint64_t* final_eval) {
  if (!ctx || !final_eval) return fail(ZK_ERR_ARG, "sparse_bool_prove: NULL argument");
  if (n_terms && (!weights || !n_positions)) return fail(ZK_ERR_ARG, "sparse_bool_prove: NULL input");
  if (num_var && (!eq_point || !round_msgs || !challenges)) return fail(ZK_ERR_ARG, "sparse_bool_prove: NULL argument");
  if (!fs && !tr) return fail(ZK_ERR_ARG, "sparse_bool_prove: neither a callback nor a transcript was given");
  uint32_t term_bits = 0;
  while ((1ull << term_bits) < n_terms) term_bits++;
  if (num_var + term_bits > 32) return fail(ZK_ERR_ARG, "sparse_bool_prove: num_var %u with %u terms exceeds the 32-bit key space", num_var, n_terms);
  // entries: every term's positions in increasing order (linear_prover.rs:497-506), key = term * 2^num_var + position;
  // the ordering runs on the device (keyset.cu)
  std::vector<uint64_t> term_begin(n_terms + 1, 0);
  for (uint32_t j = 0; j < n_terms; j++) term_begin[j + 1] = term_begin[j] + n_positions[j];
  const uint64_t total = term_begin[n_terms];
  if (total && !positions) return fail(ZK_ERR_ARG, "sparse_bool_prove: NULL positions");
  if (total >> 31) return fail(ZK_ERR_ARG, "sparse_bool_prove: too many entries");
  const uint32_t K = (uint32_t)total;

  CtxLock lk(ctx, comm != nullptr);  // a sharded call takes the first lane
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << num_var;
  char* base = nullptr;
  size_t need = al((size + size / 2 + 8) * sizeof(Fr)) + al((size / 2 * 3 + 8) * sizeof(Fr)) + al((num_var + 8) * sizeof(Fr)) + 2 * (al((K + 1) * 4ull) + al((K + 1) * sizeof(Fr))) +
                al((K / 256 + 2) * 4ull) + al((n_terms + 1) * sizeof(Fr)) + 4096;
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t o = 0;
  auto take = [&](size_t bytes) { char* p = base + o; o += al(bytes); return p; };
  Fr* eq0 = (Fr*)take((size + 1) * sizeof(Fr));
  Fr* eq1 = (Fr*)take((size / 2 + 1) * sizeof(Fr));
  Fr* eq_rec = (Fr*)take((size / 2 * 3 + 8) * sizeof(Fr));  // per-position records of the rounds after the first
  Fr* pt_dev = (Fr*)take((num_var + 8) * sizeof(Fr));
  uint32_t* e_key[2] = {(uint32_t*)take((K + 1) * 4ull), (uint32_t*)take((K + 1) * 4ull)};
  Fr* e_val[2] = {(Fr*)take((K + 1) * sizeof(Fr)), (Fr*)take((K + 1) * sizeof(Fr))};
  uint32_t* block_counts = (uint32_t*)take((K / 256 + 2) * 4ull);
  Fr* d_w = (Fr*)take((n_terms + 1) * sizeof(Fr));
  uint32_t* counts = (uint32_t*)take(256);

  if (K) {
    char* ks = nullptr;
    const size_t pos_bytes = al((size_t)K * 8), tb_bytes = al((size_t)(n_terms + 1) * 8);
    rc = ctx->reserve_aux(pos_bytes + tb_bytes + keyset_scratch_bytes(n_terms, num_var), (void**)&ks);
    if (rc) return rc;
    uint64_t* d_pos = reinterpret_cast<uint64_t*>(ks);
    uint64_t* d_tb = reinterpret_cast<uint64_t*>(ks + pos_bytes);
    ZK_CUDA(cudaMemcpyAsync(d_pos, positions, (size_t)K * 8, cudaMemcpyHostToDevice, s));
    ZK_CUDA(cudaMemcpyAsync(d_tb, term_begin.data(), (size_t)(n_terms + 1) * 8, cudaMemcpyHostToDevice, s));
    uint32_t bad[2] = {0, 0};
    rc = keyset_order(ctx, d_pos, d_tb, n_terms, K, num_var, ks + pos_bytes + tb_bytes, e_key[0], bad);
    if (rc) return rc;
    if (bad[0]) return fail(ZK_ERR_ARG, "sparse_bool_prove: position out of range in term %u", bad[0] - 1);
    if (bad[1]) return fail(ZK_ERR_ARG, "sparse_bool_prove: duplicate position in term %u", bad[1] - 1);
  }
  if (n_terms) ZK_CUDA(cudaMemcpyAsync(d_w, weights, (size_t)n_terms * sizeof(Fr), cudaMemcpyHostToDevice, s));
  ZK_CUDA(cudaMemsetAsync(counts, 0, 256, s));
  ZK_CUDA(cudaMemcpyAsync(counts, &K, 4, cudaMemcpyHostToDevice, s));
  if (K) {
    launch_fill_ones(e_val[0], K, ctx->sm_count, s);
    ctx->launches++;
  }
  // dense eq(eq_challenge, .) over the full hypercube (:509)
  rc = eq_table_device(ctx, eq_point, num_var, pt_dev, eq0);
  if (rc) return rc;
  ZK_CUDA(cudaStreamSynchronize(s));  // keys / weights host buffers may go out of scope after this

  const Fr* eq_cur = eq0;
  int e = 0;
  uint32_t k_upper = K;
  Fr challenge = Fr::zero();
  for (uint32_t round = 0; round < num_var; round++) {
    const uint32_t vars_left = num_var - round;
    const uint64_t S = 1ull << vars_left;
    // every value is one in the first round (the fill above); later rounds read the eq factors from records
    if (round) {
      launch_eq_records(eq_cur, S / 2, eq_rec, ctx->sm_count, s);
      ctx->launches++;
    }
    launch_sbool_msg(e_key[e], e_val[e], counts + e, k_upper, round ? eq_rec : eq_cur, d_w, vars_left, round == 0,
                     ctx->next_msg_scratch(comm != nullptr), s);
    ctx->launches++;
    rc = fs_round(ctx, comm, 4, round, fs, fs_user, tr, round_msgs, challenges, &challenge);
    if (rc) return rc;
    Fr* eq_next = (round & 1) ? eq0 : eq1;  // eq0 holds 2^n, eq1 2^(n-1); later rounds fit either
    launch_fold(eq_cur, eq_next, challenge, S / 2, ctx->rs.max_blocks, s);
    eq_cur = eq_next;
    ctx->launches += 1 + launch_sparse_fold(e_key[e], e_val[e], counts + e, k_upper, challenge, block_counts, e_key[e ^ 1],
                                            e_val[e ^ 1], counts + (e ^ 1), s);
    e ^= 1;
    // a term keeps at most one entry per remaining position: the bound the next round's grids are sized by
    const uint64_t cap = (uint64_t)n_terms * (S / 2);
    if (cap < k_upper) k_upper = (uint32_t)cap;
  }
  launch_sbool_final(e_key[e], e_val[e], counts + e, eq_cur, d_w, n_terms, ctx->final_out, s);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  rc = comm_sum_fr_vec(ctx, comm, ctx->final_out, 1);  // the final value is a sum over terms too
  if (rc) return rc;
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->final_out, sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  fr_store(final_eval, *reinterpret_cast<const Fr*>(ctx->host_small));
  return ZK_OK;
}

}  // namespace

extern "C" {

int zk_sumcheck_sparse_bool_prove(zk_ctx* ctx, uint32_t num_var, uint32_t n_terms, const uint64_t* weights,
                                  const uint64_t* positions, const uint64_t* n_positions, const uint64_t* eq_point,
                                  zk_fs_round_fn fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                                  uint64_t* challenges, uint64_t* final_eval) {
  return sbool_prove(ctx, nullptr, num_var, n_terms, weights, positions, n_positions, eq_point, fs, fs_user, tr, round_msgs,
                     challenges, final_eval);
}

int zk_sumcheck_sparse_bool_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t n_local_terms,
                                          const uint64_t* weights, const uint64_t* positions, const uint64_t* n_positions,
                                          const uint64_t* eq_point, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
                                          uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_eval) {
  if (!comm) return fail(ZK_ERR_ARG, "sparse_bool_prove_sharded: NULL communicator");
  // collective: after a failure on this rank the communicator is retired here, and the other ranks' bounded waits end
  return sharded_call(comm, "sparse_bool_prove_sharded", [&] {
    return sbool_prove(ctx, comm, num_var, n_local_terms, weights, positions, n_positions, eq_point, fs, fs_user, tr,
                       round_msgs, challenges, final_eval);
  });
}

int zk_sumcheck_general_prove(zk_ctx* ctx, uint32_t num_var, uint32_t num_poly, uint32_t n_terms, const uint64_t* scalars,
                              const uint64_t* const* tables, const uint64_t* eq, zk_mem mem, zk_fs_round_fn fs,
                              void* fs_user, zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                              uint64_t* final_tables, uint64_t* final_eval) {
  if (!ctx || !final_eval) return fail(ZK_ERR_ARG, "general_prove: NULL argument");
  if (n_terms == 0 || !scalars || !tables || !eq) return fail(ZK_ERR_ARG, "Polynomials cannot be empty");
  if (num_poly < 1 || num_poly > kMaxPolys + 1) return fail(ZK_ERR_ARG, "general_prove: num_poly %u out of range", num_poly);
  if (num_var > 34) return fail(ZK_ERR_ARG, "general_prove: num_var %u too large", num_var);
  if (num_var && (!round_msgs || !challenges)) return fail(ZK_ERR_ARG, "general_prove: NULL output");
  if (!fs && !tr) return fail(ZK_ERR_ARG, "general_prove: neither a callback nor a transcript was given");
  const uint32_t nf = num_poly - 1;  // factors per term; eq is the remaining one (linear_prover.rs:233)
  const uint32_t nt = n_terms * nf;
  if (nt > 256) return fail(ZK_ERR_ARG, "general_prove: at most 256 tables");
  for (uint32_t i = 0; i < nt; i++)
    if (!tables[i]) return fail(ZK_ERR_ARG, "Polynomial %u has incorrect size", i);

  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << num_var;
  const uint64_t all = (uint64_t)nt + 1;  // tables + eq
  const uint64_t in_elems = mem == ZK_MEM_HOST ? size * all : 0;
  char* base = nullptr;
  size_t need = al(in_elems * sizeof(Fr)) + al(all * (size / 2 + 1) * sizeof(Fr)) + al(all * (size / 4 + 1) * sizeof(Fr)) +
                al((n_terms + 1) * sizeof(Fr)) + al((nt + 1) * sizeof(Fr)) + 2 * al((nt + 1) * 8) + 4096;
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t o = 0;
  auto take = [&](size_t bytes) { char* p = base + o; o += al(bytes); return p; };
  Fr* in_copy = (Fr*)take(in_elems * sizeof(Fr));
  Fr* ping = (Fr*)take(all * (size / 2 + 1) * sizeof(Fr));
  Fr* pong = (Fr*)take(all * (size / 4 + 1) * sizeof(Fr));
  Fr* d_scalars = (Fr*)take((n_terms + 1) * sizeof(Fr));
  Fr* d_vals = (Fr*)take((nt + 1) * sizeof(Fr));
  const Fr** d_ptrs[2] = {(const Fr**)take((nt + 1) * 8), (const Fr**)take((nt + 1) * 8)};
  std::vector<const Fr*> cur(all);
  for (uint64_t i = 0; i < all; i++) {
    const uint64_t* src = i < nt ? tables[i] : eq;
    if (mem == ZK_MEM_HOST) {
      ZK_CUDA(cudaMemcpyAsync(in_copy + i * size, src, size * sizeof(Fr), cudaMemcpyHostToDevice, s));
      cur[i] = in_copy + i * size;
    } else {
      cur[i] = reinterpret_cast<const Fr*>(src);
    }
  }
  ZK_CUDA(cudaMemcpyAsync(d_scalars, scalars, (size_t)n_terms * sizeof(Fr), cudaMemcpyHostToDevice, s));
  Fr challenge = Fr::zero();
  for (uint32_t round = 0; round < num_var; round++) {
    const uint64_t S = size >> round;
    const Fr** dp = d_ptrs[round & 1];
    ZK_CUDA(cudaMemcpyAsync(dp, cur.data(), nt * 8, cudaMemcpyHostToDevice, s));
    launch_general_msg(dp, d_scalars, cur[nt], n_terms, nf, S / 2, ctx->next_msg_scratch(false), s);
    ctx->launches++;
    rc = fs_round(ctx, nullptr, (int)num_poly + 1, round, fs, fs_user, tr, round_msgs, challenges, &challenge);
    if (rc) return rc;
    Fr* dst = (round & 1) ? pong : ping;
    const uint64_t stride = (round & 1) ? size / 4 + 1 : size / 2 + 1;
    for (uint64_t i = 0; i < all; i++) {
      launch_fold(cur[i], dst + i * stride, challenge, S / 2, ctx->rs.max_blocks, s);
      cur[i] = dst + i * stride;
      ctx->launches++;
    }
  }
  const Fr** dp = d_ptrs[num_var & 1];
  ZK_CUDA(cudaMemcpyAsync(dp, cur.data(), nt * 8, cudaMemcpyHostToDevice, s));
  launch_general_final(dp, d_scalars, cur[nt], n_terms, nf, d_vals, ctx->final_out, s);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, ctx->final_out, sizeof(Fr), cudaMemcpyDeviceToHost, s));
  if (final_tables) ZK_CUDA(cudaMemcpyAsync(final_tables, d_vals, (size_t)nt * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  fr_store(final_eval, *reinterpret_cast<const Fr*>(ctx->host_small));
  return ZK_OK;
}

}  // extern "C"
