// Host side of the sumcheck: the verifier's round loop behind the C ABI.  No kernel is launched here; the
// file is compiled with the kernels only because it shares their field arithmetic (ff.cuh builds for the
// host as well).  SumcheckVerifier::verify, src/crypto/sumcheck/verifier.rs:27-69, with the interpolation of
// evaluate_univariate_polynomial, src/util/poly.rs:446-563 (Lagrange form over the points 0..degree).
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace zk {

// Value at x of the polynomial of degree < n_pts with the given values at 0 .. n_pts-1:
//   sum_i s(i) prod_{j != i} (x - j) / (i - j),  prod_{j != i} (i - j) = (-1)^(d-i) i! (d-i)!,  d = n_pts - 1.
Fr interpolate_at(const Fr* pts, int n_pts, const Fr& x) {
  if (n_pts <= 0) return Fr::zero();
  if (n_pts == 1) return pts[0];
  const int d = n_pts - 1;
  std::vector<Fr> diff(n_pts), fact_inv(n_pts);
  Fr f = Fr::one();
  fact_inv[0] = Fr::one();
  for (int i = 1; i <= d; i++) {
    f = mul(f, from_u32<FrParams>((uint32_t)i));
    fact_inv[i] = inverse(f);
  }
  for (int j = 0; j <= d; j++) diff[j] = sub(x, from_u32<FrParams>((uint32_t)j));
  Fr acc = Fr::zero();
  for (int i = 0; i <= d; i++) {
    Fr term = mul(pts[i], mul(fact_inv[i], fact_inv[d - i]));
    for (int j = 0; j <= d; j++)
      if (j != i) term = mul(term, diff[j]);
    acc = ((d - i) & 1) ? sub(acc, term) : add(acc, term);
  }
  return acc;
}

}  // namespace zk

extern "C" int zk_sumcheck_verify(zk_transcript* tr, uint32_t num_var, uint32_t num_poly, const uint64_t* round_msgs,
                                  uint32_t n_rounds, uint32_t msgs_per_round, const uint64_t* claimed_sum,
                                  uint64_t* challenges_out, uint64_t* final_sum_out, int* accepted,
                                  uint32_t* failed_round) {
  if (!tr || !claimed_sum || !accepted || (n_rounds && !round_msgs)) return fail(ZK_ERR_ARG, "sumcheck_verify: NULL argument");
  if (msgs_per_round > 64) return fail(ZK_ERR_ARG, "sumcheck_verify: %u evaluations per round", msgs_per_round);
  *accepted = 0;
  if (failed_round) *failed_round = 0;
  if (n_rounds != num_var) return ZK_OK;            // "Round messages length mismatch"  (verifier.rs:28-31)
  Fr running = fr_load(claimed_sum);
  for (uint32_t round = 0; round < n_rounds; round++) {
    if (failed_round) *failed_round = round;
    if (msgs_per_round != num_poly + 1) return ZK_OK;  // degree bound (:38-45)
    const uint64_t* m = round_msgs + (uint64_t)round * msgs_per_round * 4;
    Fr pts[64];
    for (uint32_t c = 0; c < msgs_per_round; c++) pts[c] = fr_load(m + 4 * c);
    if (add(pts[0], pts[1]) != running) return ZK_OK;   // (:46-54)
    for (uint32_t c = 0; c < msgs_per_round; c++) transcript_append_scalar(tr->m, (const uint8_t*)"round_message", 13, pts[c]);
    const Fr ch = transcript_challenge_scalar(tr->m, (const uint8_t*)"challenge", 9);
    running = interpolate_at(pts, (int)msgs_per_round, ch);
    if (challenges_out) fr_store(challenges_out + 4 * (uint64_t)round, ch);
  }
  if (final_sum_out) fr_store(final_sum_out, running);
  *accepted = 1;
  return ZK_OK;
}
