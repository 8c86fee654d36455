// The reference's tests/test_linear_sumcheck.rs, case by case, against the GPU prover through the
// C++ host mirror (zkes_b200/host/zkes.hpp).  Prints one line per case; exit status 0 when all pass.
#include <cstdio>
#include <functional>

#include "../../zkes_b200/host/zkes.hpp"

using namespace zkes;

static int failures = 0;
#define EXPECT(cond, msg)                                   \
  do {                                                      \
    if (!(cond)) {                                          \
      printf("  FAILED: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
      failures++;                                           \
    }                                                       \
  } while (0)

static std::vector<F> u(std::initializer_list<uint32_t> v) {
  std::vector<F> out;
  for (uint32_t x : v) out.push_back(from_u32(x));
  return out;
}

// prove on the GPU, then run the verifier with the claimed sum; returns the proof
static SumcheckProof prove_and_verify(const Context& ctx, const std::vector<std::vector<F>>& tables, size_t n, uint32_t claimed,
                                      bool expect_accept = true) {
  std::vector<DenseMLPoly> polys;
  for (const auto& t : tables) polys.push_back(DenseMLPoly::from_evaluations(t));
  Transcript transcript("sumcheck");
  LinearSumcheckProver prover(n, polys.size(), transcript);
  SumcheckProof proof = prover.prove(ctx, polys, transcript);
  EXPECT(proof.round_messages.size() == n, "one message per variable");
  for (const auto& m : proof.round_messages) EXPECT(m.size() == polys.size() + 1, "degree + 1 evaluations per round");
  Transcript vt("sumcheck");
  SumcheckVerifier verifier(n, polys.size(), vt);
  F final_sum;
  std::vector<F> ch;
  const bool ok = verifier.verify(vt, proof.round_messages, from_u32(claimed), &final_sum, &ch);
  EXPECT(ok == expect_accept, expect_accept ? "verifier accepts the honest proof" : "verifier rejects a wrong claim");
  if (ok && expect_accept) {
    EXPECT(final_sum == proof.final_eval, "final evaluation equals the verifier's running sum");
    EXPECT(ch == prover.challenges, "prover and verifier derive the same challenges");
    F prod = one();
    for (const auto& a : prover.a_arrays) prod = prod * a[0];
    EXPECT(prod == proof.final_eval, "final_eval is the product of the bound tables");
  }
  return proof;
}

int main() {
  Context ctx(0);
  struct Case { const char* name; std::function<void()> run; };
  std::vector<Case> cases = {
      {"constant_polynomials", [&] { prove_and_verify(ctx, {u({1, 1, 1, 1}), u({1, 1, 1, 1})}, 2, 4); }},          // :19-62
      {"identity_polynomials", [&] { prove_and_verify(ctx, {u({0, 1, 0, 1}), u({0, 0, 1, 1})}, 2, 1); }},          // :65-110
      {"single_variable", [&] { prove_and_verify(ctx, {u({0, 1})}, 1, 1); }},                                      // :112-134
      {"three_variables", [&] {                                                                                    // :137-182
         prove_and_verify(ctx, {u({0, 1, 1, 2, 1, 2, 2, 3}), u({0, 0, 0, 1, 0, 0, 0, 1})}, 3, 5);
       }},
      {"round_message_structure", [&] {                                                                            // :185-234
         SumcheckProof p = prove_and_verify(ctx, {u({1, 1, 1, 1}), u({0, 1, 0, 1}), u({0, 0, 1, 1})}, 2, 1);
         for (const auto& m : p.round_messages) {
           bool constant = true;
           for (const F& v : m) constant = constant && (v == m[0]);
           EXPECT(!constant, "round evaluations are not all equal");
         }
       }},
      {"zero_polynomials", [&] {                                                                                   // :237-275
         SumcheckProof p = prove_and_verify(ctx, {u({0, 0, 0, 0}), u({0, 0, 0, 0})}, 2, 0);
         for (const auto& m : p.round_messages)
           for (const F& v : m) EXPECT(v == zero(), "all-zero tables give all-zero messages");
         EXPECT(p.final_eval == zero(), "final evaluation is zero");
       }},
      {"minimal_case", [&] { prove_and_verify(ctx, {u({1, 0})}, 1, 1); }},                                         // :278-303
      {"protocol_completeness", [&] {                                                                              // :306-373
         prove_and_verify(ctx, {u({1, 2})}, 1, 3);
         prove_and_verify(ctx, {u({1, 2, 3, 4})}, 2, 10);
         prove_and_verify(ctx, {u({1, 1, 1, 1, 1, 1, 1, 1})}, 3, 8);
       }},
      {"wrong_claim_rejected", [&] { prove_and_verify(ctx, {u({1, 2, 3, 4})}, 2, 11, false); }},
      {"deterministic_behavior", [&] {                                                                             // :428-473
         SumcheckProof a = prove_and_verify(ctx, {u({3, 1, 4, 1}), u({5, 9, 2, 6})}, 2, 3 * 5 + 9 + 8 + 6);
         SumcheckProof b = prove_and_verify(ctx, {u({3, 1, 4, 1}), u({5, 9, 2, 6})}, 2, 3 * 5 + 9 + 8 + 6);
         EXPECT(a.round_messages == b.round_messages && a.final_eval == b.final_eval, "same input, same proof");
       }},
      {"shape_errors", [&] {                                                                                       // linear_prover.rs:44-52
         Transcript t("sumcheck");
         LinearSumcheckProver prover(3, 2, t);
         bool threw = false;
         try { prover.prove(ctx, {DenseMLPoly::from_evaluations(u({1, 2, 3, 4})), DenseMLPoly::from_evaluations(u({1, 2, 3, 4}))}, t); }
         catch (const std::runtime_error&) { threw = true; }
         EXPECT(threw, "wrong table size is an error");
         threw = false;
         try { prover.prove(ctx, {}, t); } catch (const std::runtime_error&) { threw = true; }
         EXPECT(threw, "no tables is an error");
       }},
      {"fix_variables_and_eq", [&] {                                                                               // test_fix_variables.rs:19-48
         DenseMLPoly f = DenseMLPoly::from_evaluations(u({1, 2, 3, 4}));
         EXPECT(f.fix_variables(ctx, u({0})).evaluations == u({1, 3}), "x0 = 0");
         EXPECT(f.fix_variables(ctx, u({1})).evaluations == u({2, 4}), "x0 = 1");
         EXPECT(fix_variables_from_right(ctx, f, u({1})).evaluations == u({3, 4}), "x1 = 1");
         EXPECT(evaluate_lagrange_basis(ctx, {}) == u({1}), "empty point");
         std::vector<F> eq = evaluate_lagrange_basis(ctx, u({1, 0, 1}));
         for (size_t i = 0; i < 8; i++) EXPECT(eq[i] == (i == 5 ? one() : zero()), "vertex indicator");
       }},
  };
  for (auto& c : cases) {
    const int before = failures;
    c.run();
    printf("%s %s\n", failures == before ? "ok  " : "FAIL", c.name);
  }
  printf("%d failure(s)\n", failures);
  return failures ? 1 : 0;
}
