/* CPU oracle (TEST INFRASTRUCTURE ONLY): multilinear helpers of src/util/poly.rs and the three
 * sumcheck provers of src/crypto/sumcheck/linear_prover.rs, restated with the same pass
 * structure (one pass over the table per evaluation point, then the fold). */
#pragma once
#include <algorithm>
#include <functional>
#include <thread>
#include <vector>
#include "transcript.h"

namespace orc {

extern int g_threads;  // worker threads used by parallel_for (set through the C API)

inline void parallel_for(size_t n, const std::function<void(size_t, size_t, int)>& fn) {
  int t = g_threads;
  if (t < 1) t = 1;
  if (n < 2048 || t == 1) {
    fn(0, n, 0);
    return;
  }
  std::vector<std::thread> th;
  const size_t chunk = (n + t - 1) / t;
  for (int i = 0; i < t; i++) {
    const size_t b = std::min(n, chunk * i), e = std::min(n, chunk * (i + 1));
    th.emplace_back([=, &fn] { fn(b, e, i); });
  }
  for (auto& x : th) x.join();
}

typedef std::vector<Fr> Table;

// evaluate_lagrange_basis / precompute_eq: util/poly.rs:573-618, 657-699
inline Table eq_table(const std::vector<Fr>& r) {
  Table a(size_t(1) << r.size(), Fr::zero());
  a[0] = Fr::one();
  for (size_t i = 0; i < r.size(); i++) {
    const size_t cur = size_t(1) << i;
    const Fr ri = r[i];
    parallel_for(cur, [&](size_t b, size_t e, int) {
      for (size_t x = b; x < e; x++) {
        const Fr hi = ri * a[x];
        a[x + cur] = hi;
        a[x] = a[x] - hi;
      }
    });
  }
  return a;
}

// one LSB fold in place: util/poly.rs:852-884, linear_prover.rs:151-178
inline void fold_in_place(Table& t, const Fr& r) {
  const size_t half = t.size() / 2;
  Table out(half);
  parallel_for(half, [&](size_t b, size_t e, int) {
    for (size_t y = b; y < e; y++) out[y] = t[2 * y] + r * (t[2 * y + 1] - t[2 * y]);
  });
  t.swap(out);
}

inline Table fix_variables(const Table& f, const std::vector<Fr>& pt) {
  Table t = f;
  for (const Fr& r : pt) fold_in_place(t, r);
  return t;
}

// fix_variables_from_right: util/poly.rs:705-758
inline Table fix_from_right(const Table& f, const std::vector<Fr>& fixed) {
  if (fixed.empty()) return f;
  size_t n = 0;
  while ((size_t(1) << n) < f.size()) n++;
  const size_t rem = n - fixed.size(), lo_n = size_t(1) << rem;
  const Table eq = eq_table(fixed);
  Table out(lo_n, Fr::zero());
  parallel_for(lo_n, [&](size_t b, size_t e, int) {
    for (size_t hi = 0; hi < eq.size(); hi++)
      for (size_t lo = b; lo < e; lo++) out[lo] = out[lo] + eq[hi] * f[hi * lo_n + lo];
  });
  return out;
}

// evaluate_multilinear_extension: util/poly.rs:622-652
inline Fr mle_eval(const Table& u, const std::vector<Fr>& r) {
  const Table eq = eq_table(r);
  Fr s = Fr::zero();
  for (size_t i = 0; i < u.size(); i++) s = s + u[i] * eq[i];
  return s;
}

struct Proof {
  std::vector<std::vector<Fr>> round_messages;
  std::vector<Fr> challenges;
  std::vector<Fr> final_tables;  // a_arrays[i][0]
  Fr final_eval;
};

// LinearSumcheckProver::prove, linear_prover.rs:43-191 (header absorbed by the caller's new()).
inline Proof linear_prove(std::vector<Table> tabs, Transcript& tr) {
  const size_t L = tabs.size();
  size_t n = 0;
  while ((size_t(1) << n) < tabs[0].size()) n++;
  Proof pf;
  for (size_t round = 0; round < n; round++) {
    const size_t half = tabs[0].size() / 2;
    std::vector<Fr> msg(L + 1);
    for (size_t c = 0; c <= L; c++) {  // one full pass per evaluation point, as the reference does
      const Fr cf = Fr::from_u64(c);
      std::vector<Fr> part(g_threads > 0 ? g_threads : 1, Fr::zero());
      parallel_for(half, [&](size_t b, size_t e, int tid) {
        Fr s = Fr::zero();
        for (size_t y = b; y < e; y++) {
          Fr g = Fr::one();
          for (size_t i = 0; i < L; i++) {
            const Fr v0 = tabs[i][2 * y], v1 = tabs[i][2 * y + 1];
            g = g * (c == 0 ? v0 : c == 1 ? v1 : v0 + cf * (v1 - v0));
          }
          s = s + g;
        }
        part[tid] = part[tid] + s;
      });
      Fr s = Fr::zero();
      for (const Fr& p : part) s = s + p;
      msg[c] = s;
    }
    for (const Fr& m : msg) tr.append_scalar("round_message", m);
    const Fr ch = tr.challenge_scalar("challenge");
    pf.round_messages.push_back(msg);
    pf.challenges.push_back(ch);
    for (auto& t : tabs) fold_in_place(t, ch);
  }
  pf.final_eval = Fr::one();
  for (auto& t : tabs) {
    pf.final_tables.push_back(t[0]);
    pf.final_eval = pf.final_eval * t[0];
  }
  return pf;
}

// SparseBoolSumcheckProver::prove, linear_prover.rs:486-656.
inline Proof sparse_bool_prove(size_t num_var, const std::vector<Fr>& weights,
                               const std::vector<std::vector<uint64_t>>& positions, const std::vector<Fr>& eq_point,
                               Transcript& tr) {
  typedef std::vector<std::pair<uint64_t, Fr>> Entries;
  std::vector<Entries> terms;
  for (auto pos : positions) {
    std::sort(pos.begin(), pos.end());
    Entries e;
    for (uint64_t p : pos) e.push_back({p, Fr::one()});
    terms.push_back(e);
  }
  Table eq = eq_table(eq_point);
  const Fr one = Fr::one(), two = Fr::from_u64(2), three = Fr::from_u64(3);
  Proof pf;
  auto walk = [](const Entries& en, size_t& i, uint64_t& rest, Fr& v0, Fr& v1) {
    const uint64_t pos = en[i].first;
    rest = pos >> 1;
    v0 = v1 = Fr::zero();
    if ((pos & 1) == 0) {
      v0 = en[i++].second;
      if (i < en.size() && en[i].first == 2 * rest + 1) v1 = en[i++].second;
    } else {
      v1 = en[i++].second;
    }
  };
  for (size_t round = 0; round < num_var; round++) {
    Fr t[4] = {Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero()};
    for (size_t j = 0; j < terms.size(); j++) {
      const Fr w = weights[j];
      for (size_t i = 0; i < terms[j].size();) {
        uint64_t rest;
        Fr v0, v1;
        walk(terms[j], i, rest, v0, v1);
        const Fr e0 = eq[2 * rest], e1 = eq[2 * rest + 1];
        t[0] = t[0] + w * v0 * (v0 - one) * e0;
        t[1] = t[1] + w * v1 * (v1 - one) * e1;
        const Fr a2 = two * v1 - v0, q2 = two * e1 - e0;
        t[2] = t[2] + w * a2 * (a2 - one) * q2;
        const Fr a3 = three * v1 - two * v0, q3 = three * e1 - two * e0;
        t[3] = t[3] + w * a3 * (a3 - one) * q3;
      }
    }
    std::vector<Fr> msg(t, t + 4);
    for (const Fr& m : msg) tr.append_scalar("round_message", m);
    const Fr ch = tr.challenge_scalar("challenge");
    pf.round_messages.push_back(msg);
    pf.challenges.push_back(ch);
    fold_in_place(eq, ch);
    for (auto& en : terms) {
      Entries ne;
      for (size_t i = 0; i < en.size();) {
        uint64_t rest;
        Fr v0, v1;
        walk(en, i, rest, v0, v1);
        const Fr nv = v0 + ch * (v1 - v0);
        if (!nv.is_zero()) ne.push_back({rest, nv});
      }
      en.swap(ne);
    }
  }
  Fr inner = Fr::zero();
  for (size_t j = 0; j < terms.size(); j++) {
    const Fr v = (!terms[j].empty() && terms[j][0].first == 0) ? terms[j][0].second : Fr::zero();
    inner = inner + weights[j] * v * (v - one);
  }
  pf.final_eval = (eq.empty() ? Fr::zero() : eq[0]) * inner;
  return pf;
}

}  // namespace orc
