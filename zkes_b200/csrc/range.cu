// Range-proof preprocessing of Dag::prove_range (src/dag/mod.rs:1314-1337), per auxiliary
// selection polynomial:
//   part[t]  = sum over the selection pairs (input_idx, table_idx = t) of eq(point)[input_idx]
//   middle   = sum_t part[t] * t
//   acc[t]  += beta_gamma * part[t]          (the running sum of the aux polynomials, :1339)
// and the table polynomial range_dense(n).add_by_scalar(alpha) (util/poly.rs:1359-1366, 915-927).
//
// The scatter-add has many pairs per table index and no order among them.  A field element has no
// atomic add, but a sum of Montgomery representations is linear: every 32-bit limb is added into
// its own 64-bit counter with one native atomic (2^32 addends cannot overflow it), and one pass
// afterwards carries the eight counters of an index into a 288-bit integer and reduces it.
#include "../../include/zkb200.h"
#include "ctx.hpp"
#include "reduce.cuh"

using namespace zk;

namespace zk {
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table);
}

namespace {

__global__ void __launch_bounds__(256) k_range_scatter(const uint64_t* __restrict__ input_idx,
                                                       const uint64_t* __restrict__ table_idx, uint64_t n_sel,
                                                       const Fr* __restrict__ eq, uint64_t n_inputs, uint64_t n_table,
                                                       unsigned long long* limbs, unsigned int* bad) {
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_sel; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t i = input_idx[e], t = table_idx[e];
    if (i >= n_inputs || t >= n_table) {
      atomicExch(bad, 1u);
      continue;
    }
    const uint4 lo = __ldg(reinterpret_cast<const uint4*>(eq + i));
    const uint4 hi = __ldg(reinterpret_cast<const uint4*>(eq + i) + 1);
    unsigned long long* L = limbs + t * 8;
    atomicAdd(L + 0, (unsigned long long)lo.x);
    atomicAdd(L + 1, (unsigned long long)lo.y);
    atomicAdd(L + 2, (unsigned long long)lo.z);
    atomicAdd(L + 3, (unsigned long long)lo.w);
    atomicAdd(L + 4, (unsigned long long)hi.x);
    atomicAdd(L + 5, (unsigned long long)hi.y);
    atomicAdd(L + 6, (unsigned long long)hi.z);
    atomicAdd(L + 7, (unsigned long long)hi.w);
  }
}

// The same for a small table (at most kSmallTable entries: lookup blocks of a few bits): with so few counters
// every global atomic would meet thousands of others on its address, so a block first adds into its own copy
// of the counters in shared memory and then flushes each non-zero counter with one global atomic.
constexpr uint32_t kSmallTable = 512;
__global__ void __launch_bounds__(256) k_range_scatter_small(const uint64_t* __restrict__ input_idx,
                                                             const uint64_t* __restrict__ table_idx, uint64_t n_sel,
                                                             const Fr* __restrict__ eq, uint64_t n_inputs, uint32_t n_table,
                                                             unsigned long long* limbs, unsigned int* bad) {
  extern __shared__ unsigned long long sh_limbs[];
  for (uint32_t k = threadIdx.x; k < n_table * 8; k += blockDim.x) sh_limbs[k] = 0;
  __syncthreads();
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_sel; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t i = input_idx[e], t = table_idx[e];
    if (i >= n_inputs || t >= n_table) {
      atomicExch(bad, 1u);
      continue;
    }
    const uint4 lo = __ldg(reinterpret_cast<const uint4*>(eq + i));
    const uint4 hi = __ldg(reinterpret_cast<const uint4*>(eq + i) + 1);
    unsigned long long* L = sh_limbs + t * 8;
    atomicAdd(L + 0, (unsigned long long)lo.x);
    atomicAdd(L + 1, (unsigned long long)lo.y);
    atomicAdd(L + 2, (unsigned long long)lo.z);
    atomicAdd(L + 3, (unsigned long long)lo.w);
    atomicAdd(L + 4, (unsigned long long)hi.x);
    atomicAdd(L + 5, (unsigned long long)hi.y);
    atomicAdd(L + 6, (unsigned long long)hi.z);
    atomicAdd(L + 7, (unsigned long long)hi.w);
  }
  __syncthreads();
  for (uint32_t k = threadIdx.x; k < n_table * 8; k += blockDim.x) {
    const unsigned long long v = sh_limbs[k];
    if (v) atomicAdd(limbs + k, v);
  }
}

// part[t] from its limb counters; acc[t] += beta_gamma * part[t]; sink.msg[0] = sum_t part[t] * t.
__global__ void __launch_bounds__(256) k_range_finish(const unsigned long long* __restrict__ limbs, uint64_t n_table,
                                                      const FixedMul<FrParams> bg, Fr* acc, const MsgSink sink) {
  Fr mid = Fr::zero();
  for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_table; t += (uint64_t)gridDim.x * blockDim.x) {
    // X = sum_j limbs[j] * 2^(32 j) < 2^288, as sixteen 32-bit limbs
    Wide x;
#pragma unroll
    for (int k = 0; k < 16; k++) x.v[k] = 0;
    unsigned long long carry = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const unsigned long long v = limbs[t * 8 + j];
      const unsigned long long s = (v & 0xffffffffull) + (carry & 0xffffffffull);
      x.v[j] = (uint32_t)s;
      carry = (v >> 32) + (carry >> 32) + (s >> 32);
    }
    x.v[8] = (uint32_t)carry;
    x.v[9] = (uint32_t)(carry >> 32);
    // X mod r in Montgomery form: redc gives X / R, one more Montgomery product by R^2 restores the factor
    const Fr part = to_mont(redc<FrParams>(x));
    Fr tt = Fr::zero();
    tt.v[0] = (uint32_t)t;
    tt.v[1] = (uint32_t)(t >> 32);
    mid = add(mid, mul(part, to_mont(tt)));
    acc[t] = add(acc[t], mul_fixed(bg, part));
  }
  Fr s[1] = {mid};
  grid_sum<1, 8>(s, sink);
}

// out[i] = i + alpha
__global__ void k_range_table(uint64_t n, const Fr alpha, Fr* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    Fr v = Fr::zero();
    v.v[0] = (uint32_t)i;
    v.v[1] = (uint32_t)(i >> 32);
    out[i] = add(to_mont(v), alpha);
  }
}

inline size_t al(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

int zk_range_aux_accumulate(zk_ctx* ctx, uint32_t k, const uint64_t* point, uint64_t n_sel, const uint64_t* input_idx,
                            const uint64_t* table_idx, zk_mem idx_mem, const uint64_t* beta_gamma, uint32_t table_log,
                            uint64_t* acc, zk_mem acc_mem, uint64_t* middle_claim_out) {
  if (!ctx || !beta_gamma || !acc || !middle_claim_out || (k && !point) || (n_sel && (!input_idx || !table_idx)))
    return fail(ZK_ERR_ARG, "range_aux_accumulate: NULL argument");
  if (k > 30 || table_log > 30) return fail(ZK_ERR_ARG, "range_aux_accumulate: k %u or table_log %u too large", k, table_log);
  if (n_sel >= (1ull << 32)) return fail(ZK_ERR_ARG, "range_aux_accumulate: at most 2^32 - 1 selection pairs");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t n_inputs = 1ull << k, n_table = 1ull << table_log;
  const bool host_idx = idx_mem == ZK_MEM_HOST, host_acc = acc_mem == ZK_MEM_HOST;
  char* base = nullptr;
  size_t need = al((n_inputs + k + 16) * sizeof(Fr)) + al(n_table * 64) + 1024;
  if (host_idx) need += 2 * al(n_sel * 8 + 8);
  if (host_acc) need += al(n_table * sizeof(Fr));
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  Fr* eq = reinterpret_cast<Fr*>(take((n_inputs + k + 16) * sizeof(Fr)));
  unsigned long long* limbs = reinterpret_cast<unsigned long long*>(take(n_table * 64));
  const uint64_t *d_in = input_idx, *d_tab = table_idx;
  if (host_idx && n_sel) {
    uint64_t* a = reinterpret_cast<uint64_t*>(take(n_sel * 8 + 8));
    uint64_t* b = reinterpret_cast<uint64_t*>(take(n_sel * 8 + 8));
    ZK_CUDA(cudaMemcpyAsync(a, input_idx, n_sel * 8, cudaMemcpyHostToDevice, s));
    ZK_CUDA(cudaMemcpyAsync(b, table_idx, n_sel * 8, cudaMemcpyHostToDevice, s));
    d_in = a;
    d_tab = b;
  }
  Fr* d_acc = reinterpret_cast<Fr*>(acc);
  if (host_acc) {
    d_acc = reinterpret_cast<Fr*>(take(n_table * sizeof(Fr)));
    ZK_CUDA(cudaMemcpyAsync(d_acc, acc, n_table * sizeof(Fr), cudaMemcpyHostToDevice, s));
  }
  rc = eq_table_device(ctx, point, k, eq + n_inputs, eq);
  if (rc) return rc;
  ZK_CUDA(cudaMemsetAsync(limbs, 0, n_table * 64, s));
  unsigned int* bad = ctx->rs.sink.counter + 14;  // spare word of the context's counter block
  ZK_CUDA(cudaMemsetAsync(bad, 0, 4, s));
  if (n_sel) {
    uint64_t blocks = (n_sel + 255) / 256;
    if (blocks > (uint64_t)ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    if (n_table <= kSmallTable) {
      if (blocks > (uint64_t)ctx->sm_count * 4) blocks = ctx->sm_count * 4;
      k_range_scatter_small<<<(unsigned)blocks, 256, n_table * 64, s>>>(d_in, d_tab, n_sel, eq, n_inputs, (uint32_t)n_table, limbs, bad);
    } else {
      k_range_scatter<<<(unsigned)blocks, 256, 0, s>>>(d_in, d_tab, n_sel, eq, n_inputs, n_table, limbs, bad);
    }
    ctx->launches++;
  }
  RoundScratch sc = ctx->rs;
  sc.sink.pub_flag = nullptr;  // read back with a copy: nothing polls this result
  uint64_t blocks = (n_table + 255) / 256;
  const uint64_t cap = (uint64_t)ctx->sm_count * 4 < (uint64_t)sc.max_blocks ? ctx->sm_count * 4 : sc.max_blocks;
  if (blocks > cap) blocks = cap;
  k_range_finish<<<(unsigned)blocks, 256, 0, s>>>(limbs, n_table, make_fixed_mul(fr_load(beta_gamma)), d_acc, sc.sink);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  char* hs = reinterpret_cast<char*>(ctx->host_small);
  ZK_CUDA(cudaMemcpyAsync(hs, ctx->rs.sink.msg, sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaMemcpyAsync(hs + 64, bad, 4, cudaMemcpyDeviceToHost, s));
  if (host_acc) ZK_CUDA(cudaMemcpyAsync(acc, d_acc, n_table * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  unsigned int was_bad = 0;
  memcpy(&was_bad, hs + 64, 4);
  if (was_bad) return fail(ZK_ERR_ARG, "range_aux_accumulate: a selection index is out of range");
  memcpy(middle_claim_out, hs, sizeof(Fr));
  return ZK_OK;
}

int zk_range_table(zk_ctx* ctx, uint32_t n, const uint64_t* alpha, uint64_t* out, zk_mem out_mem) {
  if (!ctx || !alpha || !out) return fail(ZK_ERR_ARG, "range_table: NULL argument");
  if (n > 32) return fail(ZK_ERR_ARG, "range_table: n %u too large (the reference's entries are u32)", n);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t s = ctx->stream;
  const uint64_t size = 1ull << n;
  Fr* d_out = reinterpret_cast<Fr*>(out);
  if (out_mem == ZK_MEM_HOST) {
    int rc = ctx->reserve_work(size * sizeof(Fr) + 256, (void**)&d_out);
    if (rc) return rc;
  }
  uint64_t blocks = (size + 255) / 256;
  if (blocks > (uint64_t)ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  k_range_table<<<(unsigned)blocks, 256, 0, s>>>(size, fr_load(alpha), d_out);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  if (out_mem == ZK_MEM_HOST) ZK_CUDA(cudaMemcpyAsync(out, d_out, size * sizeof(Fr), cudaMemcpyDeviceToHost, s));
  ZK_CUDA(cudaStreamSynchronize(s));
  return ZK_OK;
}

}  // extern "C"
