// Internal interface of the MSM pipeline (msm.cu) and the curve helpers kernels (curve.cu).
#pragma once
#include "ctx.hpp"
#include "ec.cuh"

namespace zk {

typedef MsmStatsPod MsmStats;

// scan.cu
uint64_t scan_scratch_elems(uint64_t n);
int exclusive_scan_u32(uint32_t* data, uint64_t n, uint32_t* scratch, bool write_total, cudaStream_t s);

// What the first pass over the scalars of an MSM finds.  A caller that runs several MSMs over the
// same scalars (C and the d_x rows of a KZH commit) passes one of these to each call: the first
// fills it, the others skip the pass.  `compact` lives in the context's compact scratch and stays
// valid until another MSM on the context analyses different scalars.
struct MsmPrep {
  bool valid = false;
  const Fr* scalars = nullptr;
  uint64_t total = 0;
  unsigned max_bits = 0;
  uint32_t max_mag = 0;            // exact largest magnitude when max_bits <= 32
  const int32_t* compact = nullptr;  // signed 32-bit form of every scalar, or NULL when some do not fit
};

// out_dev[row] = sum_i scalars[row * n + i] * bases[gather ? gather[i] : i] for row < rows.
// All pointers are device pointers; scalars are Montgomery-form Fr.  Uses the context's aux
// scratch; returns 0 or a negative status.
int msm_run(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const Fr* scalars, uint64_t n, uint32_t rows,
            Jacobian* out_dev, MsmStats* stats, MsmPrep* prep = nullptr);

int msm_run_rows(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const uint32_t* row_ids, const Fr* scalars,
                 uint64_t n, uint32_t rows, Jacobian* out_dev, MsmStats* stats, MsmPrep* prep = nullptr);

// Commitment of a selection polynomial (all listed entries one) without the digit / sort / bucket passes: msm.cu.
int msm_select_sums(zk_ctx* ctx, const Affine* full, const Affine* mid, const uint32_t* idx_dev, uint32_t n, uint32_t low_bits,
                    uint32_t rows, Jacobian* out_dev, void* scratch);

// ---- Host-side inversion.  The field code shared with the device works on 32-bit limbs, which a CPU core runs at
// about 240 ns per product, 90 us per inversion: as much as the kernels of a small commitment.  The host gets its own
// Montgomery product on 64-bit limbs (same representation: the eight 32-bit limbs read as four 64-bit ones on a
// little-endian host, R = 2^256), about 25 ns, and the inversion by Fermat on top of it.
template <class P>
struct HostMont {
  uint64_t p[4];
  uint64_t inv;  // -p^(-1) mod 2^64
  HostMont() {
    for (int i = 0; i < 4; i++) p[i] = (uint64_t)P::mod(2 * i) | ((uint64_t)P::mod(2 * i + 1) << 32);
    uint64_t x = 1;
    for (int k = 0; k < 6; k++) x *= 2 - p[0] * x;  // Newton: doubles the correct low bits each step
    inv = 0 - x;
  }
};

template <class P>
inline void host_mont_mul(const HostMont<P>& m, const uint64_t* a, const uint64_t* b, uint64_t* r) {
  typedef unsigned __int128 u128;
  uint64_t t[6] = {0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 4; i++) {
    u128 c = 0;
    for (int j = 0; j < 4; j++) {
      c += (u128)a[j] * b[i] + t[j];
      t[j] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[4] = (uint64_t)c;
    t[5] = (uint64_t)(c >> 64);
    const uint64_t q = t[0] * m.inv;
    c = ((u128)q * m.p[0] + t[0]) >> 64;
    for (int j = 1; j < 4; j++) {
      c += (u128)q * m.p[j] + t[j];
      t[j - 1] = (uint64_t)c;
      c >>= 64;
    }
    c += t[4];
    t[3] = (uint64_t)c;
    t[4] = t[5] + (uint64_t)(c >> 64);
  }
  bool ge = t[4] != 0;
  if (!ge) {
    ge = true;
    for (int j = 3; j >= 0; j--) {
      if (t[j] != m.p[j]) {
        ge = t[j] > m.p[j];
        break;
      }
    }
  }
  if (ge) {
    uint64_t borrow = 0;
    for (int j = 0; j < 4; j++) {
      const uint64_t d = t[j] - m.p[j] - borrow;
      borrow = (t[j] < m.p[j] + borrow) || (borrow && m.p[j] == ~0ull);
      t[j] = d;
    }
  }
  for (int j = 0; j < 4; j++) r[j] = t[j];
}

// a^(p-2) in Montgomery form (0 maps to 0), as inverse() computes it.
template <class P>
inline Fp<P> inverse_host(const Fp<P>& a) {
  static const HostMont<P> m;
  uint64_t x[4], r[4], e[4];
  const Fp<P> one = Fp<P>::one();
  for (int i = 0; i < 4; i++) {
    x[i] = (uint64_t)a.v[2 * i] | ((uint64_t)a.v[2 * i + 1] << 32);
    r[i] = (uint64_t)one.v[2 * i] | ((uint64_t)one.v[2 * i + 1] << 32);
    e[i] = m.p[i];
  }
  e[0] -= 2;  // both moduli end in a limb > 2
  for (int i = 3; i >= 0; i--) {
    for (int bit = 63; bit >= 0; bit--) {
      host_mont_mul(m, r, r, r);
      if ((e[i] >> bit) & 1ull) host_mont_mul(m, r, x, r);
    }
  }
  Fp<P> out;
  for (int i = 0; i < 4; i++) {
    out.v[2 * i] = (uint32_t)r[i];
    out.v[2 * i + 1] = (uint32_t)(r[i] >> 32);
  }
  return out;
}

// CurveGroup::into_affine of one point on the host: a single inversion is a chain of some 380 dependent field
// products, about 150 us for one GPU thread and about 10 us for a CPU core with the product above.
inline Affine jacobian_to_affine_host(const Jacobian& j) {
  Affine a;
  if (j.z.is_zero()) {
    a.x = Fq::zero();
    a.y = Fq::zero();
  } else {
    const Fq zi = inverse_host(j.z), zi2 = sqr(zi);
    a.x = mul(j.x, zi2);
    a.y = mul(j.y, mul(zi2, zi));
  }
  return a;
}

}  // namespace zk
