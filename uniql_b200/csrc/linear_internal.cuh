// Internal declarations shared by the W4A16 linear translation units.
#pragma once

#include "common.cuh"

namespace uniql {

struct LinearArgs {
  const void* B;
  const void* s;
  const void* bias;
  int64_t ldd;
  int64_t n, n_out, k;
  int* counters;      // zeroed ticket counters inside the caller's scratch
  float* partials;    // split-k partial sums inside the caller's scratch
  size_t partial_bytes;
  int* status_word;
};

struct GemvPlan {
  int WN, WK, S, GCH, MT, R, xs_rows;
  size_t smem;
  size_t partial_bytes;
};

// m <= 16 per launch.
GemvPlan plan_gemv(int64_t m, int64_t n, int64_t k);
int launch_gemv(const LinearArgs& a, const __half* A, int64_t lda, __half* D, int64_t m, const GemvPlan& plan,
                bool pdl, cudaStream_t stream);

// Tensor-core (tcgen05) path for m > 16.
bool gemm_tc_supported(int64_t m, int64_t n, int64_t k);
size_t gemm_tc_scratch_bytes(int64_t m, int64_t n, int64_t k);
int launch_gemm_tc(const LinearArgs& a, const __half* A, int64_t lda, __half* D, int64_t m, cudaStream_t stream);

// Hadamard transform of fp16 rows (used by the fused linear); signals dependents early when pdl is set.
int launch_hadamard(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t dim, float scale,
                    int dtype, bool pdl_trigger, cudaStream_t stream);
int hadamard_base_of(int64_t dim);   // 40/28/20/12/1, or 0 if dim is not a supported size

}  // namespace uniql
