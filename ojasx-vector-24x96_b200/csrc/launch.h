// Host-side launch entry points shared by the C ABI translation unit.
#pragma once
#include "common.cuh"

namespace ojx {

// --- linear.cu
int plan_tile_rows(int rows, int parallel_items);
int validate_linear(const LinearProblem& P);
int launch_linear(LinearProblem P, cudaStream_t stream);
int launch_linear_group(const LinearProblem* d_probs, int nprobs, int total_items, int D, cudaStream_t stream);

}  // namespace ojx
