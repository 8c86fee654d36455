// Internal interface of the MSM pipeline (msm.cu) and the curve helpers kernels (curve.cu).
#pragma once
#include "ctx.hpp"
#include "ec.cuh"

namespace zk {

typedef MsmStatsPod MsmStats;

// scan.cu
uint64_t scan_scratch_elems(uint64_t n);
int exclusive_scan_u32(uint32_t* data, uint64_t n, uint32_t* scratch, bool write_total, cudaStream_t s);

// out_dev[row] = sum_i scalars[row * n + i] * bases[gather ? gather[i] : i] for row < rows.
// All pointers are device pointers; scalars are Montgomery-form Fr.  Uses the context's aux
// scratch; returns 0 or a negative status.
int msm_run(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const Fr* scalars, uint64_t n, uint32_t rows,
            Jacobian* out_dev, MsmStats* stats);

int msm_run_rows(zk_ctx* ctx, const Affine* bases, const uint32_t* gather, const uint32_t* row_ids, const Fr* scalars,
                 uint64_t n, uint32_t rows, Jacobian* out_dev, MsmStats* stats);

}  // namespace zk
