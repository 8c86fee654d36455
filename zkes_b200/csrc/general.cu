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
// point c, where aux(c) = v0 (1 - c) + v1 c for the pair (v0, v1) of an even / odd position.
//
// Entry by entry instead of pair by pair: (a + b)^2 - (a + b) = (a^2 - a) + (b^2 - b) + 2 a b, so a pair is its two
// entries taken alone plus the cross term 2 v0 v1 c (1 - c).  An entry alone (value v on side b, nothing on the
// other side) gives, with q = v^2:
//   c = b: q - v         c = 1 - b: 0         c = 2: b ? 4q - 2v : q + v         c = 3: b ? 9q - 3v : 4q + 2v
// times eq(c): one square and three products per entry whatever its parity (no branch), against eight for a pair
// formed first.  The cross term (-4 v0 v1 eq(2) and -12 v0 v1 eq(3)) exists only where both sides are present,
// one entry in sixteen for the selection polynomials of the lookups; those entries are queued per warp and worked
// off thirty-two at a time, so that the rare case does not cost every warp its products.
//
// The eq factors come from a per-position record built once per round (k_eq_records; the table is far smaller than
// the entry list, which repeats every position once per term): an even position holds {eq(0), eq(2), 2 eq(3)}, an
// odd one {eq(1), 2 eq(2), 3 eq(3)}, so the entry's own factors are q - v, then q + v or 2q - v, then 2q + v or
// 3q - v: sums of at most four field elements, formed without reduction (they stay below 2^256, which the second
// operand of mul() may be).
//
// The entries are ordered by (term, position), so a warp that walks a contiguous span of them stays inside one term
// for thousands of entries: the weight is taken out of the inner sum and multiplied in when a lane's term changes.
//
// ONES: the first round, where every value is one (the selection polynomials are 0/1): an entry alone gives
// 2 eq(2) and 6 eq(3), a pair nothing; no value is read and nothing is multiplied but the weights.
constexpr int kPairQueue = 64;  // per warp: a batch of 32 plus what one more sweep can add

__global__ void __launch_bounds__(256) k_eq_records(const Fr* __restrict__ eq, uint64_t pairs, Fr* __restrict__ rec) {
  for (uint64_t j = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; j < pairs; j += (uint64_t)gridDim.x * blockDim.x) {
    const Fr e0 = g_ld(eq + 2 * j), e1 = g_ld(eq + 2 * j + 1);
    const Fr de = sub(e1, e0);
    const Fr e2 = add(e1, de), e3 = add(add(e1, de), de);
    Fr* out = rec + 6 * j;
    out[0] = e0;
    out[1] = e2;
    out[2] = add(e3, e3);
    out[3] = e1;
    out[4] = add(e2, e2);
    out[5] = add(add(e3, e3), e3);
  }
}

template <bool ONES>
__global__ void __launch_bounds__(kGThreads, 2) k_sbool_msg(const uint32_t* __restrict__ keys, const Fr* __restrict__ val,
                                                            const uint32_t* __restrict__ count, const Fr* __restrict__ eq,
                                                            const Fr* __restrict__ weights, uint32_t vars_left,
                                                            const MsgSink sink) {
  __shared__ uint32_t queue[ONES ? 1 : kGThreads / 32][ONES ? 1 : kPairQueue];
  const uint32_t n = *count;
  const uint32_t mask = (vars_left >= 32) ? 0xffffffffu : ((1u << vars_left) - 1u);
  // the weighted sums over all terms are touched once per term: they live in shared memory, which leaves the
  // registers to the four running sums and the products (no spills at two blocks per SM)
  __shared__ Fr s_sm[4][kGThreads];
  auto s_add = [&](int c, const Fr& x, bool negate) {
    const Fr cur = s_sm[c][threadIdx.x];
    s_sm[c][threadIdx.x] = negate ? sub(cur, x) : add(cur, x);
  };
#pragma unroll
  for (int c = 0; c < 4; c++) s_sm[c][threadIdx.x] = Fr::zero();
  Fr inner[4] = {Fr::zero(), Fr::zero(), Fr::zero(), Fr::zero()};  // the term this lane is in, without its weight
  uint32_t cur_term = 0xffffffffu;
  const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint64_t warp = (uint64_t)blockIdx.x * (kGThreads / 32) + wib;
  const uint64_t warps = (uint64_t)gridDim.x * (kGThreads / 32);
  const uint64_t span = (((uint64_t)n + warps - 1) / warps + 31) & ~31ull;  // entries per warp, a multiple of the warp width
  const uint64_t begin = warp * span, end = begin + span < n ? begin + span : n;
  uint32_t queued = 0;  // the same in every lane of the warp
  auto flush = [&](uint32_t term) {
    const Fr w = g_ld(weights + term);
    if constexpr (ONES) {
      const Fr t2 = add(inner[2], inner[2]), t3 = add(inner[3], inner[3]);
      s_add(2, mul(w, t2), false);
      s_add(3, mul(w, add(add(t3, t3), t3)), false);
      inner[2] = inner[3] = Fr::zero();
    } else {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        s_add(c, mul(w, inner[c]), false);
        inner[c] = Fr::zero();
      }
    }
  };
  // the cross terms of 32 queued pairs (or of what is left, at the end); the even position's record holds
  // eq(2) and 2 eq(3)
  auto work_off = [&](uint32_t cnt) {
    if (lane < cnt) {
      const uint32_t i = queue[ONES ? 0 : wib][ONES ? 0 : lane];
      const uint32_t key = keys[i];
      const Fr* rec = eq + 3 * (uint64_t)(key & mask);
      const Fr w = g_ld(weights + (vars_left >= 32 ? 0 : (key >> vars_left)));
      const Fr wx = mul(w, mul(g_ld(val + i), g_ld(val + i + 1)));
      const Fr a = mul(wx, g_ld(rec + 1)), b = mul(wx, g_ld(rec + 2));
      const Fr a2 = add(a, a), b2 = add(b, b);
      s_add(2, add(a2, a2), true);           // 4 v0 v1 eq(2)
      s_add(3, add(add(b2, b2), b2), true);  // 12 v0 v1 eq(3)
    }
  };
  for (uint64_t base = begin; base < end; base += 32) {
    const uint64_t i = base + lane;
    const bool valid = i < end;
    const uint32_t key = valid ? keys[i] : 0u;
    const bool odd = key & 1u;
    const uint32_t pos = key & mask;
    const uint32_t term = vars_left >= 32 ? 0 : (key >> vars_left);
    if (valid && term != cur_term) {
      if (cur_term != 0xffffffffu) flush(cur_term);
      cur_term = term;
    }
    if constexpr (ONES) {
      // alone unless the neighbour of the same pair is the next (previous) entry
      const bool lone = valid && (odd ? !(i > 0 && keys[i - 1] == key - 1) : !(i + 1 < n && keys[i + 1] == key + 1));
      if (lone) {
        const Fr e0 = g_ld(eq + (pos & ~1u)), e1 = g_ld(eq + (pos | 1u));
        const Fr de = sub(e1, e0);
        const Fr e2 = add(e1, de);
        inner[2] = add(inner[2], e2);
        inner[3] = add(inner[3], add(e2, de));
      }
    } else {
      if (valid) {
        const Fr v = g_ld(val + i);
        const Fr* rec = eq + 3 * (uint64_t)pos;
        const Fr q = mul(v, v);
        uint32_t pm[8];
#pragma unroll
        for (int k = 0; k < 8; k++) pm[k] = FrParams::mod(k);
        Fr f0, f2, f3, sv, q2, q3, t2, t3;
        sub_lazy(f0.v, q, v);                 // q - v (+ p)
        (void)sub8(sv.v, pm, v.v);            // p - v
        (void)add8(q2.v, q.v, q.v);           // 2q
        (void)add8(q3.v, q2.v, q.v);          // 3q
#pragma unroll
        for (int k = 0; k < 8; k++) {
          sv.v[k] = odd ? sv.v[k] : v.v[k];   // +v on the even side, -v on the odd one
          t2.v[k] = odd ? q2.v[k] : q.v[k];
          t3.v[k] = odd ? q3.v[k] : q2.v[k];
        }
        (void)add8(f2.v, t2.v, sv.v);         // q + v | 2q - v  (< 3p)
        (void)add8(f3.v, t3.v, sv.v);         // 2q + v | 3q - v  (< 4p < 2^256)
        const Fr same = mul(g_ld(rec), f0);
        Fr acc;
#pragma unroll
        for (int k = 0; k < 8; k++) acc.v[k] = odd ? inner[1].v[k] : inner[0].v[k];
        acc = add(acc, same);
#pragma unroll
        for (int k = 0; k < 8; k++) {
          inner[0].v[k] = odd ? inner[0].v[k] : acc.v[k];
          inner[1].v[k] = odd ? acc.v[k] : inner[1].v[k];
        }
        inner[2] = add(inner[2], mul(g_ld(rec + 1), f2));
        inner[3] = add(inner[3], mul(g_ld(rec + 2), f3));
      }
      // an even entry whose odd neighbour is present: queue the pair's cross term
      const bool pair = valid && !odd && i + 1 < n && keys[i + 1] == key + 1;
      const uint32_t m = __ballot_sync(0xffffffffu, pair);
      if (pair) queue[wib][queued + __popc(m & ((1u << lane) - 1u))] = (uint32_t)i;
      queued += __popc(m);
      __syncwarp();
      if (queued >= 32) {
        work_off(32);
        __syncwarp();
        if (lane + 32 < queued) queue[wib][lane] = queue[wib][lane + 32];  // at most 16 are left over
        queued -= 32;
        __syncwarp();
      }
    }
  }
  if constexpr (!ONES) {
    if (queued) work_off(queued);
  }
  if (cur_term != 0xffffffffu) flush(cur_term);
  Fr s[4];
#pragma unroll
  for (int c = 0; c < 4; c++) s[c] = s_sm[c][threadIdx.x];
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
                      const Fr* weights, uint32_t vars_left, bool ones, const RoundScratch& sc, cudaStream_t s) {
  if (ones)
    k_sbool_msg<true><<<g_blocks(upper, sc), kGThreads, 0, s>>>(keys, val, count, eq, weights, vars_left, sc.sink);
  else
    k_sbool_msg<false><<<g_blocks(upper, sc), kGThreads, 0, s>>>(keys, val, count, eq, weights, vars_left, sc.sink);
}
void launch_eq_records(const Fr* eq, uint64_t pairs, Fr* rec, int sm_count, cudaStream_t s) {
  const uint64_t want = (pairs + 255) / 256;
  const int blocks = (int)(want < (uint64_t)sm_count * 8 ? (want ? want : 1) : (uint64_t)sm_count * 8);
  k_eq_records<<<blocks, 256, 0, s>>>(eq, pairs, rec);
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
