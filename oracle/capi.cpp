/* CPU oracle (TEST INFRASTRUCTURE ONLY): C entry points over the restated provers so the tests
 * and the benchmark's CPU-baseline leg can drive them through ctypes.  Field elements use the
 * same wire form as the library (4 x u64 little-endian limbs, Montgomery, R = 2^256). */
#include <cstdint>
#include <string>
#include "poly.h"
#include "gen.h"

namespace orc {
int g_threads = 1;
}
using namespace orc;

static Table load_table(const uint64_t* p, size_t n) {
  Table t(n);
  memcpy(t.data(), p, n * 32);
  return t;
}
static void store_proof(const Proof& pf, uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_tables,
                        uint64_t* final_eval) {
  size_t k = 0;
  for (auto& m : pf.round_messages)
    for (auto& v : m) memcpy(round_msgs + 4 * k++, v.l, 32);
  for (size_t i = 0; i < pf.challenges.size(); i++) memcpy(challenges + 4 * i, pf.challenges[i].l, 32);
  if (final_tables)
    for (size_t i = 0; i < pf.final_tables.size(); i++) memcpy(final_tables + 4 * i, pf.final_tables[i].l, 32);
  memcpy(final_eval, pf.final_eval.l, 32);
}

extern "C" {

void orc_set_threads(int t) { g_threads = t < 1 ? 1 : t; }

// Transcript::new(label); LinearSumcheckProver::new; prove.  tail = challenge_scalar("after").
void orc_linear_prove(const char* label, uint32_t num_var, uint32_t num_poly, const uint64_t* const* tables,
                      uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_tables, uint64_t* final_eval,
                      uint64_t* tail) {
  Transcript tr(label);
  tr.append_u64("num_var", num_var);
  tr.append_u64("num_poly", num_poly);
  std::vector<Table> tabs;
  for (uint32_t i = 0; i < num_poly; i++) tabs.push_back(load_table(tables[i], size_t(1) << num_var));
  Proof pf = linear_prove(std::move(tabs), tr);
  store_proof(pf, round_msgs, challenges, final_tables, final_eval);
  if (tail) memcpy(tail, tr.challenge_scalar("after").l, 32);
}

// Sparse x dense product sumcheck, defined as the linear prover on [a.to_dense(), b].
void orc_sparse_dense_prove(const char* label, uint32_t num_var, uint64_t nnz, const uint64_t* idx,
                            const uint64_t* vals, const uint64_t* dense, uint64_t* round_msgs, uint64_t* challenges,
                            uint64_t* final_tables, uint64_t* final_eval, uint64_t* tail) {
  Transcript tr(label);
  tr.append_u64("num_var", num_var);
  tr.append_u64("num_poly", 2);
  const size_t size = size_t(1) << num_var;
  Table a(size, Fr::zero());
  for (uint64_t i = 0; i < nnz; i++) memcpy(a[idx[i]].l, vals + 4 * i, 32);
  std::vector<Table> tabs;
  tabs.push_back(std::move(a));
  tabs.push_back(load_table(dense, size));
  Proof pf = linear_prove(std::move(tabs), tr);
  store_proof(pf, round_msgs, challenges, final_tables, final_eval);
  if (tail) memcpy(tail, tr.challenge_scalar("after").l, 32);
}

// SparseBoolSumcheckProver::new + prove.  positions: concatenated per-term lists.
void orc_sparse_bool_prove(const char* label, uint32_t num_var, uint32_t n_terms, const uint64_t* weights,
                           const uint64_t* positions, const uint64_t* n_positions, const uint64_t* eq_point,
                           uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_eval, uint64_t* tail) {
  Transcript tr(label);
  tr.append_u64("num_var", num_var);
  tr.append_u64("num_poly", 3);
  std::vector<Fr> w = load_table(weights, n_terms), pt = load_table(eq_point, num_var);
  std::vector<std::vector<uint64_t>> pos(n_terms);
  size_t off = 0;
  for (uint32_t j = 0; j < n_terms; j++) {
    pos[j].assign(positions + off, positions + off + n_positions[j]);
    off += n_positions[j];
  }
  Proof pf = sparse_bool_prove(num_var, w, pos, pt, tr);
  store_proof(pf, round_msgs, challenges, nullptr, final_eval);
  if (tail) memcpy(tail, tr.challenge_scalar("after").l, 32);
}

void orc_eq_table(uint32_t k, const uint64_t* point, uint64_t* out) {
  Table t = eq_table(load_table(point, k));
  memcpy(out, t.data(), t.size() * 32);
}
void orc_fix_variables(uint32_t n, const uint64_t* evals, uint32_t k, const uint64_t* point, uint64_t* out) {
  Table t = fix_variables(load_table(evals, size_t(1) << n), load_table(point, k));
  memcpy(out, t.data(), t.size() * 32);
}
void orc_fix_from_right(uint32_t n, const uint64_t* evals, uint32_t k, const uint64_t* point, uint64_t* out) {
  Table t = fix_from_right(load_table(evals, size_t(1) << n), load_table(point, k));
  memcpy(out, t.data(), t.size() * 32);
}
void orc_mle_eval(uint32_t n, const uint64_t* evals, const uint64_t* point, uint64_t* out) {
  Fr v = mle_eval(load_table(evals, size_t(1) << n), load_table(point, n));
  memcpy(out, v.l, 32);
}

// Seeded input streams (gen.h), elements in Montgomery form.
void orc_gen_uniform_fr(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, uint64_t* out) {
  gen_uniform(seed, stream, start, count, out);
}
void orc_gen_small_fr(uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int bits, uint64_t* out) {
  gen_small(seed, stream, start, count, bits, out);
}

}  // extern "C"
