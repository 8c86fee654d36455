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

// CurveGroup::into_affine of one point on the host: a single inversion is a chain of some 380 dependent field
// products, about 150 us for one GPU thread and a few tens of microseconds for a CPU core.
inline Affine jacobian_to_affine_host(const Jacobian& j) {
  Affine a;
  if (j.z.is_zero()) {
    a.x = Fq::zero();
    a.y = Fq::zero();
  } else {
    const Fq zi = inverse(j.z), zi2 = sqr(zi);
    a.x = mul(j.x, zi2);
    a.y = mul(j.y, mul(zi2, zi));
  }
  return a;
}

}  // namespace zk
