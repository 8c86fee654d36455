// C++ host mirror of the reference's Rust interface for the proving hot path, on top of the C ABI
// (include/zkb200.h).  Names, argument meaning and error behaviour follow the crate:
//   Transcript                 src/util/transcript.rs:13-46
//   DenseMLPoly                src/util/poly.rs:764-960 (evaluations, fix_variables)
//   SumcheckProof              src/crypto/sumcheck/prover.rs:9-14
//   LinearSumcheckProver       src/crypto/sumcheck/linear_prover.rs:13-191
//   SumcheckVerifier           src/crypto/sumcheck/verifier.rs:7-70 (host arithmetic; the verifier is
//                              outside the accelerated path and is here so tests can check proofs)
//   evaluate_lagrange_basis, fix_variables_from_right   src/util/poly.rs:573-618, 705-758
// The reference panics on shape errors; here they throw std::runtime_error with the library's message.
// Field elements are zk::Fr (Montgomery limbs, the library's wire form); host arithmetic on them uses
// the same header the kernels are built from, compiled for the host.
#pragma once
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/zkb200.h"
#include "../csrc/ff.cuh"

namespace zkes {

using F = zk::Fr;

inline F zero() { return F::zero(); }
inline F one() { return F::one(); }
inline F from_u32(uint32_t v) { return zk::from_u32<zk::FrParams>(v); }  // CryptoField::from_u32
inline F operator+(const F& a, const F& b) { return zk::add(a, b); }
inline F operator-(const F& a, const F& b) { return zk::sub(a, b); }
inline F operator*(const F& a, const F& b) { return zk::mul(a, b); }

inline void check(int status, const char* what) {
  if (status != ZK_OK) throw std::runtime_error(std::string(what) + ": " + zk_last_error());
}

class Context {
 public:
  explicit Context(int device = 0) { check(zk_init(device, &ctx_), "zk_init"); }
  ~Context() { zk_free(ctx_); }
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;
  zk_ctx* get() const { return ctx_; }

 private:
  zk_ctx* ctx_ = nullptr;
};

class Transcript {
 public:
  explicit Transcript(const std::string& label) : t_(zk_transcript_new((const uint8_t*)label.data(), label.size())) {}
  Transcript(const Transcript& o) : t_(zk_transcript_clone(o.t_)) {}
  Transcript& operator=(const Transcript&) = delete;
  ~Transcript() { zk_transcript_free(t_); }
  void append_message(const std::string& label, const std::vector<uint8_t>& m) {
    zk_transcript_append_message(t_, (const uint8_t*)label.data(), label.size(), m.data(), m.size());
  }
  void append_u64(const std::string& label, uint64_t v) { zk_transcript_append_u64(t_, (const uint8_t*)label.data(), label.size(), v); }
  void append_scalar(const std::string& label, const F& s) {
    zk_transcript_append_scalar(t_, (const uint8_t*)label.data(), label.size(), reinterpret_cast<const uint64_t*>(s.v));
  }
  F challenge_scalar(const std::string& label) {
    F out;
    zk_transcript_challenge_scalar(t_, (const uint8_t*)label.data(), label.size(), reinterpret_cast<uint64_t*>(out.v));
    return out;
  }
  zk_transcript* raw() { return t_; }

 private:
  zk_transcript* t_;
};

struct DenseMLPoly {
  size_t n = 0;
  std::vector<F> evaluations;
  static DenseMLPoly from_evaluations(std::vector<F> e) {
    size_t n = 0;
    while ((size_t(1) << n) < e.size()) n++;
    if ((size_t(1) << n) != e.size()) throw std::runtime_error("Vector length must be a power of 2");
    DenseMLPoly p;
    p.n = n;
    p.evaluations = std::move(e);
    return p;
  }
  size_t len() const { return evaluations.size(); }
  bool is_empty() const { return evaluations.empty(); }
  const F& operator[](size_t i) const { return evaluations[i]; }
  DenseMLPoly fix_variables(const Context& ctx, const std::vector<F>& partial_point) const {
    if (partial_point.size() > n) throw std::runtime_error("invalid size of partial point");
    DenseMLPoly out;
    out.n = n - partial_point.size();
    out.evaluations.resize(size_t(1) << out.n);
    check(zk_fold_lsb(ctx.get(), (uint32_t)n, (const uint64_t*)evaluations.data(), ZK_MEM_HOST, (uint32_t)partial_point.size(),
                      (const uint64_t*)partial_point.data(), (uint64_t*)out.evaluations.data(), ZK_MEM_HOST), "fix_variables");
    return out;
  }
};

inline std::vector<F> evaluate_lagrange_basis(const Context& ctx, const std::vector<F>& r) {
  std::vector<F> out(size_t(1) << r.size());
  check(zk_eq_table(ctx.get(), (uint32_t)r.size(), (const uint64_t*)r.data(), (uint64_t*)out.data(), ZK_MEM_HOST), "evaluate_lagrange_basis");
  return out;
}

inline DenseMLPoly fix_variables_from_right(const Context& ctx, const DenseMLPoly& poly, const std::vector<F>& fixed_vars) {
  if (fixed_vars.size() > poly.n) throw std::runtime_error("invalid size of partial point");
  DenseMLPoly out;
  out.n = poly.n - fixed_vars.size();
  out.evaluations.resize(size_t(1) << out.n);
  check(zk_fix_from_right(ctx.get(), (uint32_t)poly.n, (const uint64_t*)poly.evaluations.data(), ZK_MEM_HOST,
                          (uint32_t)fixed_vars.size(), (const uint64_t*)fixed_vars.data(), (uint64_t*)out.evaluations.data(),
                          ZK_MEM_HOST), "fix_variables_from_right");
  return out;
}

struct SumcheckProof {
  F final_eval;
  std::vector<std::vector<F>> round_messages;
};

class LinearSumcheckProver {
 public:
  size_t num_var, num_poly;
  std::vector<F> challenges;
  std::vector<DenseMLPoly> a_arrays;  // after prove: one entry each, a_arrays[i][0]

  // ::new absorbs the instance header (linear_prover.rs:29-41)
  LinearSumcheckProver(size_t n, size_t num_polys, Transcript& transcript) : num_var(n), num_poly(num_polys) {
    transcript.append_u64("num_var", n);
    transcript.append_u64("num_poly", num_polys);
  }

  SumcheckProof prove(const Context& ctx, const std::vector<DenseMLPoly>& instances, Transcript& transcript) {
    if (instances.empty()) throw std::runtime_error("Polynomials cannot be empty");
    if (instances[0].len() != (size_t(1) << num_var)) throw std::runtime_error("Polynomials have incorrect size");
    if (instances.size() != num_poly) throw std::runtime_error("Number of polynomials mismatch");
    std::vector<const uint64_t*> ptrs;
    for (size_t i = 0; i < instances.size(); i++) {
      if (instances[i].len() != instances[0].len()) throw std::runtime_error("Polynomial " + std::to_string(i) + " has incorrect size");
      ptrs.push_back((const uint64_t*)instances[i].evaluations.data());
    }
    std::vector<F> msgs(num_var * (num_poly + 1) + 1), ch(num_var + 1), t0(num_poly);
    F fin;
    check(zk_sumcheck_linear_prove(ctx.get(), (uint32_t)num_var, (uint32_t)num_poly, ptrs.data(), ZK_MEM_HOST, nullptr, nullptr,
                                   transcript.raw(), (uint64_t*)msgs.data(), (uint64_t*)ch.data(), (uint64_t*)t0.data(),
                                   (uint64_t*)fin.v), "LinearSumcheckProver::prove");
    challenges.assign(ch.begin(), ch.begin() + num_var);
    a_arrays.clear();
    for (const F& v : t0) a_arrays.push_back(DenseMLPoly::from_evaluations({v}));
    SumcheckProof proof;
    proof.final_eval = fin;
    for (size_t r = 0; r < num_var; r++)
      proof.round_messages.emplace_back(msgs.begin() + r * (num_poly + 1), msgs.begin() + (r + 1) * (num_poly + 1));
    return proof;
  }
};

// Value at x of the polynomial through (i, points[i]), i = 0..n-1 (evaluate_univariate_polynomial, poly.rs:446-563).
inline F evaluate_univariate_polynomial(const std::vector<F>& points, const F& x) {
  const size_t n = points.size();
  F acc = zero();
  for (size_t i = 0; i < n; i++) {
    F num = one(), den = one();
    for (size_t j = 0; j < n; j++) {
      if (j == i) continue;
      num = num * (x - from_u32((uint32_t)j));
      den = den * (from_u32((uint32_t)i) - from_u32((uint32_t)j));
    }
    acc = acc + points[i] * num * zk::inverse(den);
  }
  return acc;
}

class SumcheckVerifier {
 public:
  SumcheckVerifier(size_t num_var, size_t num_poly, Transcript& transcript) : num_var_(num_var), num_poly_(num_poly) {
    transcript.append_u64("num_var", num_var);
    transcript.append_u64("num_poly", num_poly);
  }
  // Returns true and the final running sum / challenges when every round checks out (verifier.rs:27-69).
  bool verify(Transcript& transcript, const std::vector<std::vector<F>>& round_messages, const F& claimed_sum, F* final_sum,
              std::vector<F>* challenges) {
    if (round_messages.size() != num_var_) return false;
    F running = claimed_sum;
    std::vector<F> ch;
    for (const auto& msg : round_messages) {
      if (msg.size() != num_poly_ + 1) return false;
      if (msg[0] + msg[1] != running) return false;
      for (const F& m : msg) transcript.append_scalar("round_message", m);
      const F c = transcript.challenge_scalar("challenge");
      running = evaluate_univariate_polynomial(msg, c);
      ch.push_back(c);
    }
    if (final_sum) *final_sum = running;
    if (challenges) *challenges = ch;
    return true;
  }

 private:
  size_t num_var_, num_poly_;
};

}  // namespace zkes
