// Internal declarations shared by the W4A16 linear translation units.
#pragma once

#include "common.cuh"

namespace uniql {

constexpr int kMaxProj = 4;      // projections that can share one decode launch (same activations, same k)
constexpr int kFuseBlockWords = 512;   // 8-byte words per 64-column block in a fused all-reduce slot (16 rows x 32)

// Cross-GPU traffic of a decode launch (tensor parallelism).  Everything moves as 8-byte words {2 halves, epoch}
// stored into the consumer's own memory; the word is its own ready flag.
//   reduce : where a rank would store the fp16 result of a row-parallel linear it stores its partial into every rank's
//            block instead and adds up what arrived in its own block (rank order, fp32)
//   gather_out : a column-parallel launch also stores its result columns into every rank's feature area, so that the
//            next launch on each rank can read the full activation row
//   gather_in : the activations are read from this rank's feature area (bounded poll per word) instead of A
struct CommView {
  unsigned char* bufs[8];     // every rank's communication block, addressable from this GPU
  int rank, world;
  int reduce, gather_out, gather_in;
  size_t reduce_off;          // byte offset of the reduce staging area: [2 parities][world][block_cap][512] words
  size_t reduce_epoch_off;    // per-block epoch counters (u32) of the reduce area
  int64_t block_cap;          // 64-column blocks a reduce slot has room for
  size_t gather_off;          // byte offset of the feature area: [2 parities][16 rows][feat_cap / 2] words
  size_t gather_epoch_off;    // u32 gather counter of this rank (words of a call carry counter + 1; the consumer of the
                              // gathered row advances it) followed by the consumer's u32 ticket
  int64_t feat_cap;           // features (columns) a row of the feature area has room for
  int64_t col_offset;         // gather_out: global index of this launch's column 0
};

struct DecodeProjArgs {
  const void* B;
  const void* s;
  const void* bias;
  void* D;
  int64_t ldd;
  int64_t n, n_out;
};

struct DecodeArgs {
  const void* A;              // fp16 [m, k] (ignored with comm->gather_in)
  int64_t lda;
  int64_t m, k;
  int nproj;
  DecodeProjArgs proj[kMaxProj];
  int epilogue;               // UNIQL_EPILOGUE_*
  const void* residual;       // fp16 [m, n_out] added to the rounded result, or nullptr
  int64_t ldr;
  int64_t hadamard_dim;       // 0, or the size of the transform applied to the activation rows first
  int64_t k_offset;           // first feature of this launch's k range inside the transformed row (tensor parallel)
  void* scratch;              // [tickets | partial tiles | transformed activations (separate-kernel route)]
  size_t scratch_bytes;
  int* status_word;
  const CommView* comm;       // nullptr: single GPU
  int nprefetch;              // byte ranges to pull into L2 as the launch ends (weights of the launches that follow)
  const void* prefetch_ptr[4];
  size_t prefetch_bytes[4];
};

// CTA-tiled decode kernel (w4a16_gemv.cu): single-GPU launches, activations already transformed.
size_t gemv_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue);
int launch_gemv_group(const DecodeArgs& a, const __half* A, int64_t lda, cudaStream_t stream);

// m <= 16.  Scratch bytes the launch needs (tickets included).
size_t decode_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t hadamard_dim,
                            int64_t k_offset);
int launch_decode(const DecodeArgs& a, cudaStream_t stream);

struct LinearArgs {
  const void* B;
  const void* s;
  const void* bias;
  int64_t ldd;
  int64_t n, n_out, k;
  int* status_word;
};

// Tensor-core (tcgen05) path for m > 16.
bool gemm_tc_supported(int64_t m, int64_t n, int64_t k);
size_t gemm_tc_scratch_bytes(int64_t m, int64_t n, int64_t k);
int launch_gemm_tc(const LinearArgs& a, const __half* A, int64_t lda, __half* D, int64_t m, cudaStream_t stream);
// 16 < m <= 128: up to kMaxProj projections that read the same activations (same k) as one launch of the
// operand-swapped kernel; Ds[i] receives projection i (leading dimension projs[i].ldd).
bool gemm_tc_group_supported(int64_t m, int64_t k, const int64_t* n, int nproj);
int launch_gemm_tc_group(const LinearArgs* projs, void* const* Ds, int nproj, const __half* A, int64_t lda, int64_t m,
                         cudaStream_t stream);

// Hadamard transform of fp16 rows (used by the fused linear); signals dependents early when pdl is set.
int launch_hadamard(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t dim, float scale,
                    int dtype, bool pdl_trigger, cudaStream_t stream);
int hadamard_base_of(int64_t dim);   // 40/28/20/12/1, or 0 if dim is not a supported size
// fp16 rows (at most 16) read from this rank's feature area of a tensor-parallel layer (see CommView), transformed
int launch_hadamard_feat(const CommView& cv, void* y, int64_t ldy, int64_t rows, int64_t dim, float scale,
                         int* status_word, cudaStream_t stream);
// Sign rows of the base matrix: bit a' of row[a] set <=> H[a][a'] = -1 (all zero for base 1).
void hadamard_base_signs(int base, unsigned long long* rows40);

// Fills `out` from a communicator made by uniql_comm_create.
int comm_view(void* comm, CommView* out);

}  // namespace uniql
