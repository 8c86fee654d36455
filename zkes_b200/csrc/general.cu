// The two remaining provers of src/crypto/sumcheck/linear_prover.rs:
//   SparseBoolSumcheckProver (:455-656)   sum_x eq(r,x) sum_j w_j s_j(x)(s_j(x) - 1), s_j sparse
//   GeneralLinearSumcheckProver (:193-438) sum_x eq(x) sum_j a_j prod_i p_ji(x)
// Both reuse the plain fold kernel for their dense tables; the sparse one reuses the entry fold
// and compaction of sparse.cu with keys = term * 2^(remaining variables) + index, so entries of
// different terms never pair up.
#include "internal.hpp"
#include "reduce.cuh"

namespace zk {
namespace {

constexpr int kGThreads = 256;

__device__ __forceinline__ Fr g_ld(const Fr* p) {
  const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return fr_from_chunks(lo, hi);
}

// T(c), c = 0..3, over the live entries (compute_round_message, :529-591): sum_j w_j sum_y aux(aux - 1) eq at the
// point c.  The entries are ordered by (term, position), so a warp that walks a contiguous span of them stays
// inside one term for thousands of entries: the weight is taken out of the inner sum (two products per point
// instead of three) and multiplied in when a lane's term changes.
__global__ void __launch_bounds__(kGThreads, 2) k_sbool_msg(const uint32_t* __restrict__ keys, const Fr* __restrict__ val,
                                                         const uint32_t* __restrict__ count, const Fr* __restrict__ eq,
                                                         const Fr* __restrict__ weights, uint32_t vars_left,
                                                         const MsgSink sink) {
  const uint32_t n = *count;
  const uint32_t mask = (vars_left >= 32) ? 0xffffffffu : ((1u << vars_left) - 1u);
  const Fr one = Fr::one();
  Fr s[4] = {Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero()};      // weighted, all terms
  Fr inner[4] = {Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero()};  // the term this lane is in, without its weight
  uint32_t cur_term = 0xffffffffu;
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (kGThreads / 32) + (threadIdx.x >> 5);
  const uint64_t warps = (uint64_t)gridDim.x * (kGThreads / 32);
  const uint64_t span = (((uint64_t)n + warps - 1) / warps + 31) & ~31ull;  // entries per warp, a multiple of the warp width
  const uint64_t begin = warp * span, end = begin + span < n ? begin + span : n;
  for (uint64_t i = begin + lane; i < end; i += 32) {
    const uint32_t key = keys[i];
    const bool lead = (key & 1u) == 0 || i == 0 || keys[i - 1] != key - 1;
    if (!lead) continue;
    Fr v0 = Fr::zero(), v1 = Fr::zero();
    if ((key & 1u) == 0) {
      v0 = g_ld(val + i);
      if (i + 1 < n && keys[i + 1] == key + 1) v1 = g_ld(val + i + 1);
    } else {
      v1 = g_ld(val + i);
    }
    const uint32_t pos = key & mask;
    const uint32_t term = vars_left >= 32 ? 0 : (key >> vars_left);
    if (term != cur_term) {
      if (cur_term != 0xffffffffu) {
        const Fr w = g_ld(weights + cur_term);
#pragma unroll
        for (int c = 0; c < 4; c++) {
          s[c] = add(s[c], mul(w, inner[c]));
          inner[c] = Fr::zero();
        }
      }
      cur_term = term;
    }
    const Fr e0 = g_ld(eq + (pos & ~1u)), e1 = g_ld(eq + (pos | 1u));
    const Fr dv = sub(v1, v0), de = sub(e1, e0);
    Fr aux = v0, e = e0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      // aux * (aux - 1) * eq at evaluation point c
      inner[c] = add(inner[c], mul(mul(aux, sub(aux, one)), e));
      aux = add(aux, dv);
      e = add(e, de);
    }
  }
  if (cur_term != 0xffffffffu) {
    const Fr w = g_ld(weights + cur_term);
#pragma unroll
    for (int c = 0; c < 4; c++) s[c] = add(s[c], mul(w, inner[c]));
  }
  grid_sum<4, kGThreads / 32>(s, sink);
}

// final_evaluation (:644-655): eq[0] * sum_j w_j v_j (v_j - 1), v_j = the entry with key j.
__global__ void k_sbool_final(const uint32_t* keys, const Fr* val, const uint32_t* count, const Fr* eq,
                              const Fr* weights, uint32_t n_terms, Fr* out) {
  if (threadIdx.x || blockIdx.x) return;
  const uint32_t n = *count;
  const Fr one = Fr::one();
  Fr inner = Fr::zero();
  for (uint32_t i = 0; i < n; i++) {
    const uint32_t j = keys[i];
    if (j >= n_terms) continue;
    const Fr v = val[i];
    inner = add(inner, mul(weights[j], mul(v, sub(v, one))));
  }
  out[0] = mul(eq[0], inner);
}

__global__ void k_fill_ones(Fr* out, uint32_t n) {
  const Fr one = Fr::one();
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = one;
}

struct GeneralParams {
  const Fr* const* tables;  // device array: n_terms * n_factors pointers
  const Fr* scalars;        // n_terms
  const Fr* eq;
  uint32_t n_terms, n_factors;
  uint64_t pairs;
  MsgSink sink;
};

// s(c) = sum_y eq_c(y) sum_j a_j prod_i p_ji,c(y) for c = 0 .. n_factors + 1 (compute_g_value, :298-357).
__global__ void __launch_bounds__(kGThreads) k_general_msg(const GeneralParams p) {
  constexpr int kMaxEval = kMaxPolys + 2;
  Fr s[kMaxEval];
#pragma unroll
  for (int c = 0; c < kMaxEval; c++) s[c] = Fr::zero();
  const int n_eval = (int)p.n_factors + 2;
  for (uint64_t y = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; y < p.pairs; y += (uint64_t)gridDim.x * blockDim.x) {
    const Fr e0 = g_ld(p.eq + 2 * y), e1 = g_ld(p.eq + 2 * y + 1);
    const Fr de = sub(e1, e0);
    Fr inner[kMaxEval];
#pragma unroll
    for (int c = 0; c < kMaxEval; c++) inner[c] = Fr::zero();
    for (uint32_t j = 0; j < p.n_terms; j++) {
      Fr prod[kMaxEval];
      const Fr a = g_ld(p.scalars + j);
#pragma unroll
      for (int c = 0; c < kMaxEval; c++) prod[c] = a;
      for (uint32_t i = 0; i < p.n_factors; i++) {
        const Fr* t = p.tables[j * p.n_factors + i];
        const Fr v0 = g_ld(t + 2 * y), v1 = g_ld(t + 2 * y + 1);
        const Fr dv = sub(v1, v0);
        Fr v = v0;
#pragma unroll
        for (int c = 0; c < kMaxEval; c++) {
          if (c < n_eval) prod[c] = mul(prod[c], v);
          v = add(v, dv);
        }
      }
#pragma unroll
      for (int c = 0; c < kMaxEval; c++) inner[c] = add(inner[c], prod[c]);
    }
    Fr e = e0;
#pragma unroll
    for (int c = 0; c < kMaxEval; c++) {
      if (c < n_eval) s[c] = add(s[c], mul(inner[c], e));
      e = add(e, de);
    }
  }
  grid_sum<kMaxEval, kGThreads / 32>(s, p.sink);
}

// final_evaluation (:420-437): eq[0] * sum_j a_j prod_i p_ji[0]; also writes every table's value.
__global__ void k_general_final(const Fr* const* tables, const Fr* scalars, const Fr* eq, uint32_t n_terms,
                                uint32_t n_factors, Fr* table_vals, Fr* out) {
  if (threadIdx.x || blockIdx.x) return;
  Fr inner = Fr::zero();
  for (uint32_t j = 0; j < n_terms; j++) {
    Fr prod = scalars[j];
    for (uint32_t i = 0; i < n_factors; i++) {
      const Fr v = tables[j * n_factors + i][0];
      if (table_vals) table_vals[j * n_factors + i] = v;
      prod = mul(prod, v);
    }
    inner = add(inner, prod);
  }
  out[0] = mul(inner, eq[0]);
}

inline int g_blocks(uint64_t n, const RoundScratch& sc) {
  uint64_t b = (n + kGThreads - 1) / kGThreads;
  const uint64_t cap = (uint64_t)sc.sm_count * 2 < (uint64_t)sc.max_blocks ? sc.sm_count * 2 : sc.max_blocks;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (int)b;
}

}  // namespace

void launch_sbool_msg(const uint32_t* keys, const Fr* val, const uint32_t* count, uint32_t upper, const Fr* eq,
                      const Fr* weights, uint32_t vars_left, const RoundScratch& sc, cudaStream_t s) {
  k_sbool_msg<<<g_blocks(upper, sc), kGThreads, 0, s>>>(keys, val, count, eq, weights, vars_left, sc.sink);
}
void launch_sbool_final(const uint32_t* keys, const Fr* val, const uint32_t* count, const Fr* eq, const Fr* weights,
                        uint32_t n_terms, Fr* out, cudaStream_t s) {
  k_sbool_final<<<1, 32, 0, s>>>(keys, val, count, eq, weights, n_terms, out);
}
void launch_fill_ones(Fr* out, uint32_t n, int sm_count, cudaStream_t s) {
  k_fill_ones<<<sm_count * 2, 256, 0, s>>>(out, n);
}
void launch_general_msg(const Fr* const* tables_dev, const Fr* scalars, const Fr* eq, uint32_t n_terms, uint32_t n_factors,
                        uint64_t pairs, const RoundScratch& sc, cudaStream_t s) {
  GeneralParams p{tables_dev, scalars, eq, n_terms, n_factors, pairs, sc.sink};
  k_general_msg<<<g_blocks(pairs, sc), kGThreads, 0, s>>>(p);
}
void launch_general_final(const Fr* const* tables_dev, const Fr* scalars, const Fr* eq, uint32_t n_terms,
                          uint32_t n_factors, Fr* table_vals, Fr* out, cudaStream_t s) {
  k_general_final<<<1, 32, 0, s>>>(tables_dev, scalars, eq, n_terms, n_factors, table_vals, out);
}

}  // namespace zk
