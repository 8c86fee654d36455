// Declarations shared by the kernels' translation units and the C ABI layer.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "ff.cuh"

namespace zk {

constexpr int kMaxPolys = 4;  // tables per product term the dense round kernel is built for

// Device scratch every round launch needs (owned by the context).
struct RoundScratch {
  Fr* partials;           // max_blocks * (kMaxPolys + 1) elements
  unsigned int* counter;  // zero between launches
  Fr* msg;                // kMaxPolys + 1 elements: the round message
  int max_blocks;         // capacity of partials, in blocks
  int sm_count;
};

// sumcheck.cu
void launch_round(int num_poly, bool fold, const Fr* const* src, Fr* const* dst, const Fr& r, uint64_t pairs,
                  const RoundScratch& sc, cudaStream_t stream);
void launch_final(int num_poly, bool bind, const Fr* const* src, const Fr& r, Fr* out, cudaStream_t stream);
void launch_fold(const Fr* src, Fr* dst, const Fr& r, uint64_t out_len, int max_blocks, cudaStream_t stream);

}  // namespace zk
