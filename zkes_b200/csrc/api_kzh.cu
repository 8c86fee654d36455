// C ABI: KZH2 / KZH3 structured reference strings, commit and open (G1 side).
#include "../../include/zkb200.h"
#include "msm.hpp"
#include "kzh.hpp"

#include <vector>

using namespace zk;

namespace zk {
size_t fixed_base_table_bytes();
int fixed_base_build_table(const Affine& g, void* table_mem, cudaStream_t s);
int fixed_base_generate(const void* table_mem, int n_factors, const Fr* const* tables, const uint32_t* bits,
                        const Fr* alpha, uint64_t start, uint64_t count, Affine* out, int sm_count, cudaStream_t s);
int comm_sum_points(zk_ctx* ctx, zk_comm* c, Jacobian* point);
int comm_sum_fr_vec(zk_ctx* ctx, zk_comm* c, Fr* vals, uint64_t n);
int normalize_device(zk_ctx* ctx, const Jacobian* in, uint64_t n, Affine* out);
size_t from_right_scratch_elems(zk_ctx* ctx, uint32_t n, uint32_t k);
int fix_from_right_device(zk_ctx* ctx, uint32_t n, const Fr* f_dev, uint32_t k, const uint64_t* point_host, Fr* scratch,
                          Fr* out_dev);
int eq_table_device(zk_ctx* ctx, const uint64_t* point_host, uint32_t k, Fr* point_dev, Fr* table);
}  // namespace zk

namespace {

inline size_t al(size_t x) { return (x + 255) & ~(size_t)255; }

// get_degree_from_maximum_supported_degree: kzh2.rs:423-429, kzh3.rs:429-437
void split_degrees(int dims, uint32_t n, uint32_t* x, uint32_t* y, uint32_t* z) {
  if (dims == 2) {
    *x = n / 2;
    *y = n - n / 2;
    *z = 0;
  } else {
    const uint32_t k = n / 3;
    *x = k + (n % 3 >= 1);
    *y = k + (n % 3 == 2);
    *z = k;
  }
}

int alloc_srs(zk_ctx* ctx, int dims, uint32_t n, int rank, int world, zk_kzh_srs** out) {
  if (!ctx || !out) return fail(ZK_ERR_ARG, "kzh_srs: NULL argument");
  if (dims != 2 && dims != 3) return fail(ZK_ERR_ARG, "kzh_srs: dims must be 2 or 3");
  if (n > 30) return fail(ZK_ERR_ARG, "kzh_srs: n %u too large", n);
  cudaSetDevice(ctx->device);
  zk_kzh_srs* s = new zk_kzh_srs();
  s->dims = dims;
  s->n = n;
  split_degrees(dims, n, &s->x_log, &s->y_log, &s->z_log);
  if (world < 1 || (world & (world - 1)) || rank < 0 || rank >= world || (uint64_t)world > (1ull << s->x_log)) {
    delete s;
    return fail(ZK_ERR_ARG, "kzh_srs: %d ranks cannot share 2^%u rows", world, s->x_log);
  }
  s->rank = rank;
  s->world = world;
  s->count[0] = (1ull << n) / world;
  s->slab_begin = s->count[0] * rank;
  s->count[1] = 1ull << (n - s->x_log);
  s->count[2] = dims == 3 ? 1ull << s->z_log : 0;
  for (int k = 0; k < 3; k++) {
    if (!s->count[k]) continue;
    cudaError_t e = cudaMalloc(&s->h[k], s->count[k] * sizeof(Affine));
    if (e != cudaSuccess) {
      cudaGetLastError();
      for (int j = 0; j < 3; j++) cudaFree(s->h[j]);
      delete s;
      return fail(ZK_ERR_OOM, "kzh_srs: %llu points: %s", (unsigned long long)(1ull << n), cudaGetErrorString(e));
    }
  }
  *out = s;
  return ZK_OK;
}

// Device copy of the evaluations, zero-extended to 2^n (extend_number_of_variables, poly.rs:925-938).
int stage_poly(zk_ctx* ctx, uint32_t n, uint32_t poly_n, const uint64_t* evals, zk_mem mem, Fr* staging, const Fr** f) {
  const uint64_t size = 1ull << n, have = 1ull << poly_n;
  if (mem == ZK_MEM_DEVICE && poly_n == n) {
    *f = reinterpret_cast<const Fr*>(evals);
    return ZK_OK;
  }
  ZK_CUDA(cudaMemcpyAsync(staging, evals, have * sizeof(Fr), cudaMemcpyDefault, ctx->stream));
  if (have < size) ZK_CUDA(cudaMemsetAsync(staging + have, 0, (size - have) * sizeof(Fr), ctx->stream));
  *f = staging;
  return ZK_OK;
}

// split_input (kzh2.rs:479-498, kzh3.rs:443-460): left-pad with zeros to n coordinates.
void pad_point(const uint64_t* point, uint32_t point_len, uint32_t n, std::vector<uint64_t>& out) {
  out.assign((size_t)n * 4, 0);
  if (point_len >= n) {
    if (n) memcpy(out.data(), point, (size_t)n * 32);  // longer inputs: the leading coordinates are used
  } else if (point_len) {
    memcpy(out.data() + (size_t)(n - point_len) * 4, point, (size_t)point_len * 32);
  }
}

// Everything of kzh3_open after f_prime (kzh3.rs:739-779), shared by the whole-table and the
// sharded entry points; scratch is kzh3_tail_bytes() of device memory.
size_t kzh3_tail_bytes(zk_ctx* ctx, const zk_kzh_srs* srs) {
  const uint64_t nx = 1ull << srs->x_log, ny = 1ull << srs->y_log, nz = 1ull << srs->z_log;
  return al(nz * sizeof(Fr)) + al((nx + 8) * sizeof(Fr)) * 2 +
         al(from_right_scratch_elems(ctx, srs->y_log + srs->z_log, srs->y_log) * sizeof(Fr)) + al((nx + 2) * sizeof(Jacobian)) +
         al((ny + 2) * sizeof(Jacobian)) + al((nx + 1) * sizeof(Affine)) + 2048;
}

int kzh3_open_tail(zk_ctx* ctx, const zk_kzh_srs* srs, const Fr* f_prime, const std::vector<uint64_t>& pt,
                   const uint64_t* d_x_jac, char* mem, uint64_t* d_y_jac_out, uint64_t* c_y_affine_out, uint64_t* f_star_out) {
  cudaStream_t st = ctx->stream;
  const uint32_t xl = srs->x_log, yl = srs->y_log, zl = srs->z_log;
  const uint64_t nx = 1ull << xl, ny = 1ull << yl, nz = 1ull << zl;
  const uint64_t* r_y = pt.data() + (size_t)zl * 4;
  const uint64_t* r_x = pt.data() + (size_t)(zl + yl) * 4;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = mem + off; off += al(bytes); return p; };
  Fr* f_star = (Fr*)take(nz * sizeof(Fr));
  Fr* eq_x = (Fr*)take((nx + 8) * sizeof(Fr));
  Fr* pt_dev = (Fr*)take((nx + 8) * sizeof(Fr));
  Fr* scratch = (Fr*)take(from_right_scratch_elems(ctx, yl + zl, yl) * sizeof(Fr));
  Jacobian* d_dx = (Jacobian*)take((nx + 2) * sizeof(Jacobian));
  Jacobian* d_dy = (Jacobian*)take((ny + 2) * sizeof(Jacobian));
  Affine* d_aff = (Affine*)take((nx + 1) * sizeof(Affine));
  // d_y[i] = MSM(h_z, f_prime[i * 2^z_log ..])   (kzh3.rs:743-750)
  ctx->prof_begin(ZK_PROF_MSM, 0.0, 8);
  int rc = msm_run(ctx, srs->h[2], nullptr, f_prime, nz, (uint32_t)ny, d_dy, nullptr);
  ctx->prof_end();
  if (rc) return rc;
  // f_star = fix_variables_from_right(poly, r_y || r_x) = fix_variables_from_right(f_prime, r_y)   (kzh3.rs:762-764)
  if (yl == 0) {
    ZK_CUDA(cudaMemcpyAsync(f_star, f_prime, nz * sizeof(Fr), cudaMemcpyDeviceToDevice, st));
  } else {
    rc = fix_from_right_device(ctx, yl + zl, f_prime, yl, r_y, scratch, f_star);
    if (rc) return rc;
  }
  // c_y = MSM(affine(d_x), eq(r_x))   (kzh3.rs:739, 767-779)
  ZK_CUDA(cudaMemcpyAsync(d_dx, d_x_jac, nx * sizeof(Jacobian), cudaMemcpyHostToDevice, st));
  rc = normalize_device(ctx, d_dx, nx, d_aff);
  if (rc) return rc;
  rc = eq_table_device(ctx, r_x, xl, pt_dev, eq_x);
  if (rc) return rc;
  ctx->prof_begin(ZK_PROF_MSM, 0.0, 8);
  rc = msm_run(ctx, d_aff, nullptr, eq_x, nx, 1, d_dy + ny, &ctx->last_msm);
  ctx->prof_end();
  if (rc) return rc;
  rc = normalize_device(ctx, d_dy + ny, 1, d_aff + nx);
  if (rc) return rc;
  ZK_CUDA(cudaMemcpyAsync(d_y_jac_out, d_dy, ny * sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(c_y_affine_out, d_aff + nx, sizeof(Affine), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(f_star_out, f_star, nz * sizeof(Fr), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  return ZK_OK;
}

// ---- opening of a sparse polynomial: the contraction over x runs over the non-zero entries only
// (sparse_kzh2.rs:99-116, sparse_kzh3.rs:140-170):  out[lo] = sum over entries (idx = hi * 2^low_bits + lo, v)
// of eq(r_x)[hi] * v.  Entries that share `lo` meet in no particular order; a field element has no atomic add,
// but a sum of Montgomery representations is linear, so every 32-bit limb of a term goes into its own 64-bit
// counter with one native atomic, and a second pass carries and reduces the eight counters of an output.
__global__ void __launch_bounds__(256) k_sparse_contract(const uint64_t* __restrict__ idx, const Fr* __restrict__ vals,
                                                         uint64_t nnz, uint32_t low_bits, uint64_t limit,
                                                         const Fr* __restrict__ eq, unsigned long long* limbs, unsigned int* bad) {
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t i = idx[e];
    if (i >= limit) {
      atomicExch(bad, 1u);
      continue;
    }
    Fr w = eq[i >> low_bits];
    if (vals) w = mul(w, vals[e]);
    unsigned long long* L = limbs + (i & ((1ull << low_bits) - 1)) * 8;
#pragma unroll
    for (int k = 0; k < 8; k++) atomicAdd(L + k, (unsigned long long)w.v[k]);
  }
}

__global__ void __launch_bounds__(256) k_limbs_to_fr(const unsigned long long* __restrict__ limbs, uint64_t n, Fr* out) {
  for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (uint64_t)gridDim.x * blockDim.x) {
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
    out[t] = to_mont(redc<FrParams>(x));  // X mod r: redc gives X / R, the product by R^2 restores the factor
  }
}

// f_prime (device, 2^(n - x_log) elements) of a sparse polynomial.  mem: sparse_contract_bytes() of device memory.
size_t sparse_contract_bytes(const zk_kzh_srs* srs, uint64_t nnz, bool with_vals) {
  const uint64_t nx = 1ull << srs->x_log, lo_n = 1ull << (srs->n - srs->x_log);
  return al(nnz * 8 + 8) + (with_vals ? al(nnz * sizeof(Fr) + 32) : 0) + al((nx + srs->x_log + 16) * sizeof(Fr)) + al(lo_n * 64) + 512;
}

int sparse_contract_x(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                      const uint64_t* r_x, char* mem, Fr* f_prime) {
  cudaStream_t st = ctx->stream;
  const uint32_t xl = srs->x_log, low_bits = srs->n - xl;
  const uint64_t nx = 1ull << xl, lo_n = 1ull << low_bits;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = mem + off; off += al(bytes); return p; };
  uint64_t* d_idx = (uint64_t*)take(nnz * 8 + 8);
  Fr* d_val = vals ? (Fr*)take(nnz * sizeof(Fr) + 32) : nullptr;
  Fr* eq = (Fr*)take((nx + xl + 16) * sizeof(Fr));
  unsigned long long* limbs = (unsigned long long*)take(lo_n * 64);
  unsigned int* bad = ctx->rs.sink.counter + 16;
  if (nnz) {
    ZK_CUDA(cudaMemcpyAsync(d_idx, indices, nnz * 8, cudaMemcpyHostToDevice, st));
    if (vals) ZK_CUDA(cudaMemcpyAsync(d_val, vals, nnz * sizeof(Fr), cudaMemcpyHostToDevice, st));
  }
  int rc = eq_table_device(ctx, r_x, xl, eq + nx, eq);
  if (rc) return rc;
  ZK_CUDA(cudaMemsetAsync(limbs, 0, lo_n * 64, st));
  ZK_CUDA(cudaMemsetAsync(bad, 0, 4, st));
  if (nnz) {
    uint64_t blocks = (nnz + 255) / 256;
    if (blocks > (uint64_t)ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    k_sparse_contract<<<(unsigned)blocks, 256, 0, st>>>(d_idx, d_val, nnz, low_bits, 1ull << srs->n, eq, limbs, bad);
    ctx->launches++;
  }
  uint64_t blocks = (lo_n + 255) / 256;
  if (blocks > (uint64_t)ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  k_limbs_to_fr<<<(unsigned)blocks, 256, 0, st>>>(limbs, lo_n, f_prime);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  return ZK_OK;
}

}  // namespace

extern "C" {

int zk_kzh_srs_setup_sharded(zk_ctx* ctx, int rank, int world, int dims, uint32_t n, const uint64_t* g_affine,
                             const uint64_t* tau_x, const uint64_t* tau_y, const uint64_t* tau_z, const uint64_t* alpha,
                             zk_kzh_srs** out);

int zk_kzh_srs_setup(zk_ctx* ctx, int dims, uint32_t n, const uint64_t* g_affine, const uint64_t* tau_x,
                     const uint64_t* tau_y, const uint64_t* tau_z, const uint64_t* alpha, zk_kzh_srs** out) {
  return zk_kzh_srs_setup_sharded(ctx, 0, 1, dims, n, g_affine, tau_x, tau_y, tau_z, alpha, out);
}

int zk_kzh_srs_setup_sharded(zk_ctx* ctx, int rank, int world, int dims, uint32_t n, const uint64_t* g_affine,
                             const uint64_t* tau_x, const uint64_t* tau_y, const uint64_t* tau_z, const uint64_t* alpha,
                             zk_kzh_srs** out) {
  if (!g_affine || !tau_x || !tau_y) return fail(ZK_ERR_ARG, "kzh_srs_setup: NULL argument");
  if (dims == 2 && !alpha) return fail(ZK_ERR_ARG, "kzh_srs_setup: KZH2 needs alpha");
  if (dims == 3 && !tau_z) return fail(ZK_ERR_ARG, "kzh_srs_setup: KZH3 needs tau_z");
  zk_kzh_srs* s = nullptr;
  int rc = alloc_srs(ctx, dims, n, rank, world, &s);
  if (rc) return rc;
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint64_t nx = 1ull << s->x_log, ny = 1ull << s->y_log, nz = dims == 3 ? 1ull << s->z_log : 0;
  char* base = nullptr;
  rc = ctx->reserve_aux(fixed_base_table_bytes() + al((nx + ny + nz + 4) * sizeof(Fr)) + 1024, (void**)&base);
  if (rc) { cudaFree(s->h[0]); cudaFree(s->h[1]); cudaFree(s->h[2]); delete s; return rc; }
  void* table = base;
  Fr* d_tx = reinterpret_cast<Fr*>(base + al(fixed_base_table_bytes()));
  Fr* d_ty = d_tx + nx;
  Fr* d_tz = d_ty + ny;
  ZK_CUDA(cudaMemcpyAsync(d_tx, tau_x, nx * sizeof(Fr), cudaMemcpyHostToDevice, st));
  ZK_CUDA(cudaMemcpyAsync(d_ty, tau_y, ny * sizeof(Fr), cudaMemcpyHostToDevice, st));
  if (nz) ZK_CUDA(cudaMemcpyAsync(d_tz, tau_z, nz * sizeof(Fr), cudaMemcpyHostToDevice, st));
  Affine g;
  memcpy(&g, g_affine, sizeof(Affine));
  ctx->launches += fixed_base_build_table(g, table, st);
  if (dims == 2) {
    // h_xy[i] = (tau_x[x] tau_y[y]) g with y in the low bits; h_y[j] = (alpha tau_y[j]) g   (kzh2.rs:521-541)
    const Fr* t2[2] = {d_ty, d_tx};
    const uint32_t b2[2] = {s->y_log, s->x_log};
    ctx->launches += fixed_base_generate(table, 2, t2, b2, nullptr, s->slab_begin, s->count[0], s->h[0], ctx->sm_count, st);
    Fr a = fr_load(alpha);
    const Fr* t1[1] = {d_ty};
    const uint32_t b1[1] = {s->y_log};
    ctx->launches += fixed_base_generate(table, 1, t1, b1, &a, 0, s->count[1], s->h[1], ctx->sm_count, st);
  } else {
    // h_xyz (z low, y middle, x high), h_yz, h_z   (kzh3.rs:480-531)
    const Fr* t3[3] = {d_tz, d_ty, d_tx};
    const uint32_t b3[3] = {s->z_log, s->y_log, s->x_log};
    ctx->launches += fixed_base_generate(table, 3, t3, b3, nullptr, s->slab_begin, s->count[0], s->h[0], ctx->sm_count, st);
    ctx->launches += fixed_base_generate(table, 2, t3, b3, nullptr, 0, s->count[1], s->h[1], ctx->sm_count, st);
    ctx->launches += fixed_base_generate(table, 1, t3, b3, nullptr, 0, s->count[2], s->h[2], ctx->sm_count, st);
  }
  ZK_CUDA(cudaGetLastError());
  ZK_CUDA(cudaStreamSynchronize(st));
  *out = s;
  return ZK_OK;
}

int zk_kzh_srs_upload(zk_ctx* ctx, int dims, uint32_t n, const uint64_t* h_full, const uint64_t* h_mid,
                      const uint64_t* h_low, zk_mem mem, zk_kzh_srs** out) {
  if (!h_full || !h_mid || (dims == 3 && !h_low)) return fail(ZK_ERR_ARG, "kzh_srs_upload: NULL argument");
  zk_kzh_srs* s = nullptr;
  int rc = alloc_srs(ctx, dims, n, 0, 1, &s);
  if (rc) return rc;
  CtxLock lk(ctx);
  ctx = lk.lane;
  const uint64_t* src[3] = {h_full, h_mid, h_low};
  for (int k = 0; k < 3; k++)
    if (s->count[k]) ZK_CUDA(cudaMemcpyAsync(s->h[k], src[k], s->count[k] * sizeof(Affine), cudaMemcpyDefault, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  (void)mem;
  *out = s;
  return ZK_OK;
}

void zk_kzh_srs_free(zk_ctx* ctx, zk_kzh_srs* srs) {
  if (!srs) return;
  if (ctx) {
    CtxLock lk(ctx);
  ctx = lk.lane;
    cudaStreamSynchronize(ctx->stream);
    for (int k = 0; k < 3; k++) cudaFree(srs->h[k]);
  }
  delete srs;
}

int zk_kzh_srs_shape(const zk_kzh_srs* srs, uint32_t* x_log, uint32_t* y_log, uint32_t* z_log) {
  if (!srs) return fail(ZK_ERR_ARG, "kzh_srs_shape: NULL srs");
  if (x_log) *x_log = srs->x_log;
  if (y_log) *y_log = srs->y_log;
  if (z_log) *z_log = srs->z_log;
  return ZK_OK;
}

int zk_kzh_srs_read(zk_ctx* ctx, const zk_kzh_srs* srs, int which, uint64_t offset, uint64_t count, uint64_t* out) {
  if (!ctx || !srs || !out || which < 0 || which > 2) return fail(ZK_ERR_ARG, "kzh_srs_read: bad argument");
  if (offset + count > srs->count[which]) return fail(ZK_ERR_ARG, "kzh_srs_read: range past the end");
  CtxLock lk(ctx);
  ctx = lk.lane;
  ZK_CUDA(cudaMemcpyAsync(out, srs->h[which] + offset, count * sizeof(Affine), cudaMemcpyDeviceToHost, ctx->stream));
  ZK_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZK_OK;
}

int zk_kzh_commit(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                  uint64_t* c_affine_out, uint64_t* d_x_jac_out) {
  if (!ctx || !srs || !evals || !c_affine_out || !d_x_jac_out) return fail(ZK_ERR_ARG, "kzh_commit: NULL argument");
  if (poly_n > srs->n) return fail(ZK_ERR_ARG, "Cannot extend to fewer variables");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint32_t n = srs->n;
  const uint64_t size = 1ull << n, rows = 1ull << srs->x_log;
  char* base = nullptr;
  int rc = ctx->reserve_work(al(size * sizeof(Fr)) + al((rows + 1) * sizeof(Jacobian)) + al(sizeof(Affine)) + 1024, (void**)&base);
  if (rc) return rc;
  Fr* staging = reinterpret_cast<Fr*>(base);
  Jacobian* d_jac = reinterpret_cast<Jacobian*>(base + al(size * sizeof(Fr)));
  Affine* d_c = reinterpret_cast<Affine*>(base + al(size * sizeof(Fr)) + al((rows + 1) * sizeof(Jacobian)));
  const Fr* f = nullptr;
  rc = stage_poly(ctx, n, poly_n, evals, evals_mem, staging, &f);
  if (rc) return rc;
  // C = sum_i f[i] h_full[i]   (kzh2.rs:636-647, kzh3.rs:662-673)
  MsmPrep prep;  // both MSMs run over the same scalars: one analysis pass serves the two
  ctx->prof_begin(ZK_PROF_MSM, 0.0, 8);
  rc = msm_run(ctx, srs->h[0], nullptr, f, size, 1, d_jac + rows, &ctx->last_msm, &prep);
  ctx->prof_end();
  if (rc) return rc;
  // d_x[i] = sum_j f[i * 2^(n - x_log) + j] h_mid[j]   (kzh2.rs:653-660, kzh3.rs:680-687)
  ctx->prof_begin(ZK_PROF_MSM, 0.0, 8);
  rc = msm_run(ctx, srs->h[1], nullptr, f, srs->count[1], (uint32_t)rows, d_jac, nullptr, &prep);
  ctx->prof_end();
  if (rc) return rc;
  Jacobian* h_c = reinterpret_cast<Jacobian*>(reinterpret_cast<char*>(ctx->host_small) + 4096);
  ZK_CUDA(cudaMemcpyAsync(h_c, d_jac + rows, sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(d_x_jac_out, d_jac, rows * sizeof(Jacobian), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  const Affine c_aff = jacobian_to_affine_host(*h_c);  // the commitment's affine form (into_affine)
  memcpy(c_affine_out, &c_aff, sizeof(Affine));
  return ZK_OK;
}

int zk_kzh2_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                 const uint64_t* point, uint32_t point_len, uint64_t* f_star_out) {
  if (!ctx || !srs || !evals || !f_star_out || (point_len && !point)) return fail(ZK_ERR_ARG, "kzh2_open: NULL argument");
  if (srs->dims != 2) return fail(ZK_ERR_ARG, "kzh2_open: the SRS is not a KZH2 SRS");
  if (poly_n > srs->n) return fail(ZK_ERR_ARG, "Cannot extend to fewer variables");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint32_t n = srs->n;
  const uint64_t size = 1ull << n, ny = 1ull << srs->y_log;
  std::vector<uint64_t> pt;
  pad_point(point, point_len, n, pt);
  char* base = nullptr;
  int rc = ctx->reserve_work(al(size * sizeof(Fr)) + al(ny * sizeof(Fr)) +
                             al(from_right_scratch_elems(ctx, n, srs->x_log) * sizeof(Fr)) + 1024, (void**)&base);
  if (rc) return rc;
  Fr* staging = reinterpret_cast<Fr*>(base);
  Fr* d_out = reinterpret_cast<Fr*>(base + al(size * sizeof(Fr)));
  Fr* scratch = reinterpret_cast<Fr*>(base + al(size * sizeof(Fr)) + al(ny * sizeof(Fr)));
  const Fr* f = nullptr;
  rc = stage_poly(ctx, n, poly_n, evals, evals_mem, staging, &f);
  if (rc) return rc;
  // f_star = fix_variables_from_right(poly, r_x), r_x = the x_log highest coordinates (kzh2.rs:700-704)
  if (srs->x_log == 0) {
    ZK_CUDA(cudaMemcpyAsync(d_out, f, ny * sizeof(Fr), cudaMemcpyDeviceToDevice, st));
  } else {
    rc = fix_from_right_device(ctx, n, f, srs->x_log, pt.data() + (size_t)srs->y_log * 4, scratch, d_out);
    if (rc) return rc;
  }
  ZK_CUDA(cudaMemcpyAsync(f_star_out, d_out, ny * sizeof(Fr), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  return ZK_OK;
}

int zk_kzh3_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                 const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                 uint64_t* c_y_affine_out, uint64_t* f_star_out) {
  if (!ctx || !srs || !evals || !d_x_jac || !d_y_jac_out || !c_y_affine_out || !f_star_out || (point_len && !point))
    return fail(ZK_ERR_ARG, "kzh3_open: NULL argument");
  if (srs->dims != 3) return fail(ZK_ERR_ARG, "kzh3_open: the SRS is not a KZH3 SRS");
  if (poly_n > srs->n) return fail(ZK_ERR_ARG, "Cannot extend to fewer variables");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint32_t n = srs->n, xl = srs->x_log;
  const uint64_t size = 1ull << n, nyz = 1ull << (srs->y_log + srs->z_log);
  std::vector<uint64_t> pt;
  pad_point(point, point_len, n, pt);
  const uint64_t* r_x = pt.data() + (size_t)(srs->z_log + srs->y_log) * 4;
  const size_t fr_scr = from_right_scratch_elems(ctx, n, xl);
  char* base = nullptr;
  int rc = ctx->reserve_work(al(size * sizeof(Fr)) + al(nyz * sizeof(Fr)) + al(fr_scr * sizeof(Fr)) + kzh3_tail_bytes(ctx, srs),
                             (void**)&base);
  if (rc) return rc;
  Fr* staging = (Fr*)base;
  Fr* f_prime = (Fr*)(base + al(size * sizeof(Fr)));
  Fr* scratch = (Fr*)(base + al(size * sizeof(Fr)) + al(nyz * sizeof(Fr)));
  char* tail_mem = base + al(size * sizeof(Fr)) + al(nyz * sizeof(Fr)) + al(fr_scr * sizeof(Fr));
  const Fr* f = nullptr;
  rc = stage_poly(ctx, n, poly_n, evals, evals_mem, staging, &f);
  if (rc) return rc;
  // f_prime = fix_variables_from_right(poly, r_x)   (kzh3.rs:736)
  if (xl == 0) {
    ZK_CUDA(cudaMemcpyAsync(f_prime, f, nyz * sizeof(Fr), cudaMemcpyDeviceToDevice, st));
  } else {
    rc = fix_from_right_device(ctx, n, f, xl, r_x, scratch, f_prime);
    if (rc) return rc;
  }
  return kzh3_open_tail(ctx, srs, f_prime, pt, d_x_jac, tail_mem, d_y_jac_out, c_y_affine_out, f_star_out);
}

// kzh2_open / kzh3_open over a table sharded by x-rows (the layout of zk_kzh_commit_sharded): every
// rank contracts its slab with its slice of eq(r_x), the partial tables are summed over the ranks,
// and the small remainder of the opening (d_y, f_star, c_y) is computed on every rank alike.
static int kzh_open_sharded_impl(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals, zk_mem evals_mem,
                        const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                        uint64_t* c_y_affine_out, uint64_t* f_star_out) {
  if (!ctx || !comm || !srs || !local_evals || !f_star_out || (point_len && !point))
    return fail(ZK_ERR_ARG, "kzh_open_sharded: NULL argument");
  const bool k3 = srs->dims == 3;
  if (k3 && (!d_x_jac || !d_y_jac_out || !c_y_affine_out)) return fail(ZK_ERR_ARG, "kzh_open_sharded: a KZH3 opening needs d_x, d_y and c_y");
  const int world = comm_world(comm), rank = comm_rank(comm);
  if (world != srs->world || rank != srs->rank) return fail(ZK_ERR_ARG, "kzh_open_sharded: the SRS was set up for rank %d of %d", srs->rank, srs->world);
  CtxLock lk(ctx, true);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint32_t n = srs->n, xl = srs->x_log;
  const uint64_t lo_n = 1ull << (n - xl), hi_n = 1ull << xl, hi_local = hi_n / world, slab = hi_local * lo_n;
  std::vector<uint64_t> pt;
  pad_point(point, point_len, n, pt);
  const uint64_t* r_x = pt.data() + (size_t)(n - xl) * 4;
  const uint32_t splits = from_right_splits(lo_n, hi_local, ctx->sm_count);
  char* base = nullptr;
  size_t need = al((xl + 8) * sizeof(Fr)) + al(hi_n * sizeof(Fr)) + al((size_t)splits * lo_n * sizeof(Fr)) + al(lo_n * sizeof(Fr)) +
                (evals_mem == ZK_MEM_HOST ? al(slab * sizeof(Fr)) : 0) + (k3 ? kzh3_tail_bytes(ctx, srs) : 0) + 1024;
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  Fr* pt_dev = (Fr*)take((xl + 8) * sizeof(Fr));
  Fr* eq = (Fr*)take(hi_n * sizeof(Fr));
  Fr* partial = (Fr*)take((size_t)splits * lo_n * sizeof(Fr));
  Fr* f_prime = (Fr*)take(lo_n * sizeof(Fr));
  const Fr* f = reinterpret_cast<const Fr*>(local_evals);
  if (evals_mem == ZK_MEM_HOST) {
    Fr* p = (Fr*)take(slab * sizeof(Fr));
    ZK_CUDA(cudaMemcpyAsync(p, local_evals, slab * sizeof(Fr), cudaMemcpyHostToDevice, st));
    f = p;
  }
  char* tail_mem = k3 ? take(kzh3_tail_bytes(ctx, srs)) : nullptr;
  rc = eq_table_device(ctx, r_x, xl, pt_dev, eq);
  if (rc) return rc;
  ctx->launches += launch_from_right(f, eq + hi_local * rank, lo_n, hi_local, partial, f_prime, ctx->sm_count, st);
  rc = comm_sum_fr_vec(ctx, comm, f_prime, lo_n);
  if (rc) return rc;
  ZK_CUDA(cudaGetLastError());
  if (!k3) {  // f_star = fix_variables_from_right(poly, r_x)   (kzh2.rs:700-704)
    ZK_CUDA(cudaMemcpyAsync(f_star_out, f_prime, lo_n * sizeof(Fr), cudaMemcpyDeviceToHost, st));
    ZK_CUDA(cudaStreamSynchronize(st));
    return ZK_OK;
  }
  return kzh3_open_tail(ctx, srs, f_prime, pt, d_x_jac, tail_mem, d_y_jac_out, c_y_affine_out, f_star_out);
}

int zk_kzh_open_sharded(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals, zk_mem evals_mem,
                        const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                        uint64_t* c_y_affine_out, uint64_t* f_star_out) {
  if (!comm) return fail(ZK_ERR_ARG, "kzh_open_sharded: NULL communicator");
  return sharded_call(comm, "kzh_open_sharded", [&] { return kzh_open_sharded_impl(ctx, comm, srs, local_evals, evals_mem, point, point_len, d_x_jac, d_y_jac_out, c_y_affine_out, f_star_out); });
}

// The G1 and field checks of kzh2_verify (kzh2.rs:763-789: steps 2 and 3) and kzh3_verify
// (kzh3.rs:836-886: checks 2, 4 and 5); the pairing checks stay with the caller.
int zk_kzh_verify_g1(zk_ctx* ctx, const zk_kzh_srs* srs, const uint64_t* point, uint32_t point_len, const uint64_t* output,
                     const uint64_t* d_x_jac, const uint64_t* d_y_jac, const uint64_t* c_y_affine, const uint64_t* f_star,
                     int* ok, int* failed_check) {
  if (!ctx || !srs || !output || !d_x_jac || !f_star || !ok || (point_len && !point))
    return fail(ZK_ERR_ARG, "kzh_verify_g1: NULL argument");
  if (srs->dims == 3 && (!d_y_jac || !c_y_affine)) return fail(ZK_ERR_ARG, "kzh_verify_g1: a KZH3 opening carries d_y and c_y");
  if (srs->world != 1) return fail(ZK_ERR_ARG, "kzh_verify_g1: needs a whole (unsharded) SRS");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const bool k3 = srs->dims == 3;
  const uint32_t n = srs->n, xl = srs->x_log, yl = srs->y_log, zl = srs->z_log;
  const uint32_t low_log = k3 ? zl : yl;                  // variables of f_star
  const uint64_t nx = 1ull << xl, ny = 1ull << yl, n_low = 1ull << low_log;
  std::vector<uint64_t> pt;
  pad_point(point, point_len, n, pt);
  const uint64_t* r_low = pt.data();                                  // r_y (KZH2) or r_z (KZH3)
  const uint64_t* r_y3 = pt.data() + (size_t)zl * 4;                  // KZH3 only
  const uint64_t* r_x = pt.data() + (size_t)(k3 ? zl + yl : yl) * 4;
  const uint64_t n_big = nx > ny ? nx : ny;
  char* base = nullptr;
  size_t need = al((n_big + 1) * sizeof(Jacobian)) + al((n_big + 1) * sizeof(Affine)) + al((n_big + 40) * sizeof(Fr)) * 2 +
                al(n_low * sizeof(Fr)) * 2 + al(8 * sizeof(Jacobian)) + al(8 * sizeof(Affine)) + 2048;
  int rc = ctx->reserve_work(need, (void**)&base);
  if (rc) return rc;
  size_t off = 0;
  auto take = [&](size_t bytes) { char* p = base + off; off += al(bytes); return p; };
  Jacobian* d_jac = (Jacobian*)take((n_big + 1) * sizeof(Jacobian));
  Affine* d_aff = (Affine*)take((n_big + 1) * sizeof(Affine));
  Fr* eq = (Fr*)take((n_big + 40) * sizeof(Fr));
  Fr* pt_dev = (Fr*)take((n_big + 40) * sizeof(Fr));
  Fr* d_fstar = (Fr*)take(n_low * sizeof(Fr));
  Fr* eq_low = (Fr*)take(n_low * sizeof(Fr));
  Jacobian* res = (Jacobian*)take(8 * sizeof(Jacobian));
  Affine* res_aff = (Affine*)take(8 * sizeof(Affine));

  // res[0] = MSM(affine(d_x), eq(r_x))
  ZK_CUDA(cudaMemcpyAsync(d_jac, d_x_jac, nx * sizeof(Jacobian), cudaMemcpyHostToDevice, st));
  rc = normalize_device(ctx, d_jac, nx, d_aff);
  if (rc) return rc;
  rc = eq_table_device(ctx, r_x, xl, pt_dev, eq);
  if (rc) return rc;
  rc = msm_run(ctx, d_aff, nullptr, eq, nx, 1, res + 0, nullptr);
  if (rc) return rc;
  // res[1] = MSM(h_low, f_star)
  ZK_CUDA(cudaMemcpyAsync(d_fstar, f_star, n_low * sizeof(Fr), cudaMemcpyHostToDevice, st));
  rc = msm_run(ctx, srs->h[k3 ? 2 : 1], nullptr, d_fstar, n_low, 1, res + 1, nullptr);
  if (rc) return rc;
  if (k3) {  // res[2] = MSM(affine(d_y), eq(r_y))
    ZK_CUDA(cudaMemcpyAsync(d_jac, d_y_jac, ny * sizeof(Jacobian), cudaMemcpyHostToDevice, st));
    rc = normalize_device(ctx, d_jac, ny, d_aff);
    if (rc) return rc;
    rc = eq_table_device(ctx, r_y3, yl, pt_dev, eq);
    if (rc) return rc;
    rc = msm_run(ctx, d_aff, nullptr, eq, ny, 1, res + 2, nullptr);
    if (rc) return rc;
  }
  rc = normalize_device(ctx, res, k3 ? 3 : 2, res_aff);
  if (rc) return rc;
  // f_star(r_low)
  rc = eq_table_device(ctx, r_low, low_log, pt_dev, eq_low);
  if (rc) return rc;
  RoundScratch sc = ctx->rs;
  sc.sink.pub_flag = nullptr;
  launch_dot(d_fstar, eq_low, n_low, sc, st);
  ctx->launches++;
  ZK_CUDA(cudaGetLastError());
  char* h = reinterpret_cast<char*>(ctx->host_small);
  ZK_CUDA(cudaMemcpyAsync(h, res_aff, 3 * sizeof(Affine), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(h + 256, ctx->rs.sink.msg, sizeof(Fr), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  const char* a0 = h;                    // sum eq(r_x)[i] d_x[i]
  const char* a1 = h + sizeof(Affine);   // MSM(h_low, f_star)
  const char* a2 = h + 2 * sizeof(Affine);
  int bad = 0;
  if (!k3) {
    if (memcmp(a0, a1, sizeof(Affine)) != 0) bad = 2;
    else if (memcmp(h + 256, output, sizeof(Fr)) != 0) bad = 3;
  } else {
    if (memcmp(a0, c_y_affine, sizeof(Affine)) != 0) bad = 2;
    else if (memcmp(a1, a2, sizeof(Affine)) != 0) bad = 4;
    else if (memcmp(h + 256, output, sizeof(Fr)) != 0) bad = 5;
  }
  *ok = bad == 0;
  if (failed_check) *failed_check = bad;
  return ZK_OK;
}

// sparse_kzh2_open (sparse_kzh2.rs:84-127): same point convention as the dense open (split_input, :97-98).
int zk_sparse_kzh2_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                        const uint64_t* point, uint32_t point_len, uint64_t* f_star_out) {
  if (!ctx || !srs || !f_star_out || (nnz && !indices) || (point_len && !point)) return fail(ZK_ERR_ARG, "sparse_kzh2_open: NULL argument");
  if (srs->dims != 2) return fail(ZK_ERR_ARG, "sparse_kzh2_open: the SRS is not a KZH2 SRS");
  if (srs->world != 1) return fail(ZK_ERR_ARG, "sparse_kzh2_open: needs an unsharded SRS");
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint64_t ny = 1ull << srs->y_log;
  std::vector<uint64_t> pt;
  pad_point(point, point_len, srs->n, pt);
  char* base = nullptr;
  int rc = ctx->reserve_work(sparse_contract_bytes(srs, nnz, vals != nullptr) + al(ny * sizeof(Fr)) + 1024, (void**)&base);
  if (rc) return rc;
  Fr* f_star = reinterpret_cast<Fr*>(base);
  rc = sparse_contract_x(ctx, srs, nnz, indices, vals, pt.data() + (size_t)srs->y_log * 4, base + al(ny * sizeof(Fr)), f_star);
  if (rc) return rc;
  unsigned int* bad = ctx->rs.sink.counter + 16;
  ZK_CUDA(cudaMemcpyAsync(f_star_out, f_star, ny * sizeof(Fr), cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, bad, 4, cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  if (*reinterpret_cast<const unsigned int*>(ctx->host_small)) return fail(ZK_ERR_ARG, "sparse_kzh2_open: an index is outside the SRS domain");
  return ZK_OK;
}

// sparse_kzh3_open (sparse_kzh3.rs:112-232); a short point is padded with trailing zeros here (:124-131), unlike
// the dense open.
int zk_sparse_kzh3_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                        const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                        uint64_t* c_y_affine_out, uint64_t* f_star_out) {
  if (!ctx || !srs || (nnz && !indices) || (point_len && !point) || !d_x_jac || !d_y_jac_out || !c_y_affine_out || !f_star_out)
    return fail(ZK_ERR_ARG, "sparse_kzh3_open: NULL argument");
  if (srs->dims != 3) return fail(ZK_ERR_ARG, "sparse_kzh3_open: the SRS is not a KZH3 SRS");
  if (srs->world != 1) return fail(ZK_ERR_ARG, "sparse_kzh3_open: needs an unsharded SRS");
  std::vector<uint64_t> pt((size_t)srs->n * 4, 0);
  const uint32_t take_n = point_len < srs->n ? point_len : srs->n;
  if (take_n) memcpy(pt.data(), point, (size_t)take_n * 32);
  CtxLock lk(ctx);
  ctx = lk.lane;
  cudaStream_t st = ctx->stream;
  const uint64_t nyz = 1ull << (srs->y_log + srs->z_log);
  char* base = nullptr;
  int rc = ctx->reserve_work(sparse_contract_bytes(srs, nnz, vals != nullptr) + al(nyz * sizeof(Fr)) + kzh3_tail_bytes(ctx, srs) + 1024,
                             (void**)&base);
  if (rc) return rc;
  Fr* f_prime = reinterpret_cast<Fr*>(base);
  char* tail_mem = base + al(nyz * sizeof(Fr));
  char* contract_mem = tail_mem + kzh3_tail_bytes(ctx, srs);
  rc = sparse_contract_x(ctx, srs, nnz, indices, vals, pt.data() + (size_t)(srs->y_log + srs->z_log) * 4, contract_mem, f_prime);
  if (rc) return rc;
  unsigned int* bad = ctx->rs.sink.counter + 16;
  ZK_CUDA(cudaMemcpyAsync(ctx->host_small, bad, 4, cudaMemcpyDeviceToHost, st));
  ZK_CUDA(cudaStreamSynchronize(st));
  if (*reinterpret_cast<const unsigned int*>(ctx->host_small)) return fail(ZK_ERR_ARG, "sparse_kzh3_open: an index is outside the SRS domain");
  return kzh3_open_tail(ctx, srs, f_prime, pt, d_x_jac, tail_mem, d_y_jac_out, c_y_affine_out, f_star_out);
}

}  // extern "C"
