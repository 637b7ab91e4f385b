// Internal declarations shared by the W4A16 linear translation units.
#pragma once

#include "common.cuh"

namespace uniql {

// Optional cross-GPU sum fused into the decode kernel's epilogue (row-parallel linears): where each rank would
// store its fp16 partial, it stores {2 halves, epoch} words into every rank's staging block instead and then
// sums the words that arrived in its own block.
struct ArFuse {
  unsigned char* bufs[8];     // every rank's communication block, addressable from this GPU
  int rank, world;
  size_t staging_off;         // byte offset of the fused staging area inside a block
  size_t epoch_off;           // byte offset of the per-column-group epoch counters
  int64_t words_per_slot;     // 8-byte words per (parity, source rank) slot
  int enabled;
};

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
  const ArFuse* ar;   // nullptr: plain store
};

struct GemvPlan {
  int WN, WK, S, GCH, MT, R, xs_rows;
  int cluster, ctile_off;
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
int hadamard_base_of(int64_t dim);

// Fills `out` from a communicator made by uniql_comm_create; fails if m*n does not fit its staging area.
int comm_fuse_desc(void* comm, int64_t m, int64_t n, ArFuse* out);   // 40/28/20/12/1, or 0 if dim is not a supported size

}  // namespace uniql
