/*
 * uniql_b200 — C ABI of the B200 (sm_100a) kernels behind UniQL's W4A16 hot path.
 *
 * Plain pointers and sizes only; no torch types.  All pointers are DEVICE
 * pointers unless a comment says otherwise.  Every function enqueues work on
 * `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream)
 * and returns without synchronising.  Return value: 0 on success, a negative
 * UNIQL_E* code otherwise (nothing was enqueued in that case).  No function
 * allocates device memory unless its comment says so; scratch is supplied by
 * the caller.  Nothing throws across this boundary.
 *
 * Reference citations are paths inside the UniQL project.
 */
#ifndef UNIQL_B200_H_
#define UNIQL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UNIQL_ABI_VERSION 2

enum {
  UNIQL_OK = 0,
  UNIQL_EINVAL = -1,       /* null pointer, negative size, misaligned pointer          */
  UNIQL_EGROUPSIZE = -2,   /* groupsize other than 128 (per-channel mode unsupported)   */
  UNIQL_ESHAPE = -3,       /* n % 64 != 0, k % 128 != 0, dim not a supported size, ...  */
  UNIQL_ESCRATCH = -4,     /* scratch buffer missing or too small                       */
  UNIQL_ECUDA = -5,        /* a CUDA runtime call failed (see uniql_last_cuda_error)    */
  UNIQL_EDTYPE = -6,       /* unsupported element type code                             */
  UNIQL_ESTATIC = -7       /* problem needs more than the built-in scratch of uniql_w4a16_linear_static */
};

/* Element type codes for uniql_hadamard. */
enum { UNIQL_F16 = 0, UNIQL_BF16 = 1, UNIQL_F32 = 2 };

/* Bits that kernels OR into *status_word (device int, may be NULL). */
enum {
  UNIQL_STATUS_BAD_TOKEN_ID = 1,  /* an embedding id was outside [0, vocab); row written as zeros */
  UNIQL_STATUS_WAIT_TIMEOUT = 2,  /* a bounded wait (asynchronous copy, or words another GPU has to write) gave up;
                                     the output is invalid */
  UNIQL_STATUS_BAD_INDEX = 4      /* a slicing index pointed outside the source layer; that column / row was written as zeros */
};

int uniql_abi_version(void);
const char* uniql_strerror(int code);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread. */
int uniql_last_cuda_error(void);

/*
 * W4A16 linear forward:  D[m, 0:n_out] = A[m, k] * dequant(B, s) (+ bias), fp32 accumulation, fp16 output.
 * Replaces quant_linear_cuda.w4a16o16_gemm (csrc/linear/quant_linear.cpp:6-24, host wrapper
 * csrc/linear/marlin_gemm_kernel.cuh:991-1052) and the bias add / padding slice of
 * W4A16B16O16Linear.forward (quantize/quant_linear_layers.py:91-116).
 *
 *   A          fp16 [m, k], row stride lda elements (lda >= k, rows 16-byte aligned)
 *   B          int32 [k/16, 2*n] packed int4 in the reference's permuted order
 *              (quantize/quantize_helpers.py:145-165, 67-84)
 *   s          fp16 [k/128, n] group scales in the reference's permuted order (:54-62, 169-180)
 *   bias       fp16 [n_out] or NULL
 *   D          fp16 [m, n_out], row stride ldd elements
 *   n          stored (padded) output width, multiple of 64; n_out <= n columns are written
 *   k          multiple of 128
 *   groupsize  128; -1 (per-channel) returns UNIQL_EGROUPSIZE
 *   hadamard_dim  0, or k: apply y = H_k * x / sqrt(k) to every row of A first
 *              (quantize/quant_hadamard_layers.py:16-18 placed in front of the linear);
 *              the transformed rows are rounded to fp16 exactly as the separate module would.
 *              The transform runs as a few-row kernel in front of the linear, which starts as its programmatic
 *              dependent (its weight stream overlaps the transform); the slot-balanced decode kernel
 *              (UNIQL_B200_DECODE_ENGINE=slot) runs it inside its own prologue for m <= 4.
 *   scratch    device buffer of at least uniql_w4a16_scratch_bytes(m, n, k, hadamard_dim) bytes,
 *              256-byte aligned.  Its first UNIQL_SCRATCH_COUNTER_BYTES bytes must be zero before the
 *              first call and are left zero by every call; do not share one scratch buffer between
 *              calls that may overlap on the GPU.
 *   status_word  optional device int for kernel-side diagnostics (unused bits stay untouched)
 */
#define UNIQL_SCRATCH_COUNTER_BYTES 16384
int uniql_w4a16_linear(const void* A, int64_t lda, const void* B, const void* s, const void* bias,
                       void* D, int64_t ldd, int64_t m, int64_t n, int64_t n_out, int64_t k,
                       int groupsize, int64_t hadamard_dim, void* scratch, size_t scratch_bytes,
                       int* status_word, void* stream);

/* Scratch requirement of uniql_w4a16_linear for this problem on the current device. */
size_t uniql_w4a16_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t hadamard_dim);

/*
 * Decode-size W4A16 linear (m <= 16, no Hadamard) for callers that have no way to hand over device scratch.
 * This entry point has no counterpart in the reference.  It exists for hosts that may not allocate device
 * memory at the point where they call into this library: a plugin running inside someone else's memory
 * plan, a real-time loop that forbids allocator calls after start-up, code that only receives the tensors of
 * the op and nothing else.  Same arguments and results as uniql_w4a16_linear minus the scratch pointer; the
 * split-k counters and partial sums live in a UNIQL_STATIC_SCRATCH_BYTES array inside the library image
 * instead (every GPU that loads the library keeps that much memory until the process exits).
 *
 *  - Nothing is allocated or freed, by this function or by anything it calls.
 *  - Problems whose partial sums do not fit the array are refused with UNIQL_ESTATIC (nothing is enqueued);
 *    m > 16 returns UNIQL_ESHAPE.  uniql_w4a16_scratch_bytes(m, n, k, 0) tells what a problem needs.
 *  - The first call on each device looks up the array's device address and clears its counter region
 *    (one memset enqueued on `stream`); make that first call outside of any stream capture.
 *  - All calls on a device share the one array, and it keeps whatever the last call left in it (the counters
 *    are always left at zero).  Two calls that can run at the same time on the GPU (different streams) would
 *    race on it: serialise them.
 */
#define UNIQL_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int uniql_w4a16_linear_static(const void* A, int64_t lda, const void* B, const void* s, const void* bias,
                              void* D, int64_t ldd, int64_t m, int64_t n, int64_t n_out, int64_t k,
                              int groupsize, int* status_word, void* stream);

/*
 * 4-bit embedding gather: out[t, :] = fp16((q - 8) * scales[ids[t]]), bit-exact with
 * quant_embedding_cuda.w4a16_embedding_lookup (csrc/embedding/quant_embedding.cpp:3-8,
 * kernel csrc/embedding/quant_embedding_kernel.cuh:47-114).
 *
 *   ids     int64 [n_ids]
 *   W       int32 [vocab, dim/8]  (quantize/quant_embedding_layers.py:33-43 packing)
 *   scales  fp16 [vocab]
 *   out     fp16 [n_ids, dim]
 *   dim     multiple of 8
 * An id outside [0, vocab) writes a zero row and sets UNIQL_STATUS_BAD_TOKEN_ID in *status_word
 * (the reference reads out of bounds there).
 */
int uniql_w4_embedding(const int64_t* ids, int64_t n_ids, const void* W, const void* scales,
                       void* out, int64_t vocab, int64_t dim, int* status_word, void* stream);

/*
 * Hadamard transform along the last axis: y[r, :] = (H_dim x[r, :]) * scale.
 * Replaces fast_hadamard_transform_cuda.fast_hadamard_transform{,_12N,_20N,_28N,_40N}
 * (call sites quantize/hadamard_helpers.py:18-48).  dim = base * 2^j with base chosen in the
 * reference's order 40, 28, 20, 12, else 1 (power of two).  x and y may alias.
 *   dtype  UNIQL_F16 / UNIQL_BF16 / UNIQL_F32 (both x and y); arithmetic is fp32.
 */
int uniql_hadamard(const void* x, void* y, int64_t rows, int64_t dim, float scale, int dtype, void* stream);

/*
 * Round-to-nearest group-128 int4 quantiser + packer on the GPU: fp16 nn.Linear weight -> the `weight` / `scale`
 * buffers of W4A16B16O16Linear, bit-identical to the reference's CPU path.
 * Replaces W4A16B16O16Linear.from_fp16's call of w4a16_quantize(W^T, 4, 128, scale, pad_out)
 * (quantize/quant_linear_layers.py:50-89, quantize/quantize_helpers.py:184-241 with :88-141, :145-180).
 *   W            fp16 [n_out, k_in] row-major with row stride ldw (elements): the nn.Linear layout, no transpose needed
 *   group_scale  NULL for RTN (s = max|w| * 2/15 per group and column); or fp16 [ceil(k_in/128), n_out] in natural
 *                column order when the weight is already fake-quantised on those scales (the GPTQ hand-over, :205-218)
 *   packed       out, int32 [Kp/16, 2*n_pad], Kp = k_in rounded up to 128 (k rows past k_in quantise zeros)
 *   scales       out, fp16 [Kp/128, n_pad], permuted inside 64-column blocks
 *   w_ref        out or NULL, fp16 [Kp, n_pad]: the dequantised weights the reference returns alongside
 *   n_pad        stored column count: a multiple of 64, >= n_out (the reference uses the next multiple of 256);
 *                columns past n_out get code 0, scale 0
 */
int uniql_w4a16_quantize(const void* W, int64_t ldw, int64_t n_out, int64_t k_in, const void* group_scale,
                         void* packed, void* scales, void* w_ref, int64_t n_pad, void* stream);

/*
 * Load-time slicing of packed layers on the GPU (the reference re-slices on the CPU through unpack -> slice -> repack:
 * modeling/modeling_helpers.py:361-867 with quantize/quantize_helpers.py:279-328 and :67-84).
 *
 * uniql_w4a16_gather_columns: new packed layer whose output column c is source column col_index[c] (c < n_new; the
 * columns from n_new to n_out_pad, and entries < 0, get code 0 and scale 0).  Rows k >= zero_rows_from get code 0 (the
 * reference drops the k padding before slicing and pads with zeros afterwards); pass size_k to keep every row.
 *   packed_in  int32 [size_k/16, 2*n_src_pad]   scales_in  fp16 [size_k/128, n_src_pad] (permuted)
 *   packed_out int32 [size_k/16, 2*n_out_pad]   scales_out fp16 [size_k/128, n_out_pad] (permuted)
 *   col_index  DEVICE int32 [n_new], values in [0, n_src_pad) or negative; a value >= n_src_pad is treated like a
 *              negative one and raises UNIQL_STATUS_BAD_INDEX in *status_word (device int, may be NULL)
 *
 * uniql_w4a16_dequantize_rows: out[n][j] = fp16((q - 8) * s) of source row row_index[j], column n, for n < n_real and
 * j < k_new, row stride ld (elements): the [out_features, in_features] layout uniql_w4a16_quantize reads, so that
 * "keep these input rows and quantise again" (slice_w4a16_o_proj :632-650, slice_w4a16_out_proj :845-862) is two calls.
 *   row_index  DEVICE int32 [k_new], values in [0, size_k); any other value writes zeros for that row and raises
 *              UNIQL_STATUS_BAD_INDEX in *status_word
 */
int uniql_w4a16_gather_columns(const void* packed_in, const void* scales_in, int64_t size_k, int64_t n_src_pad,
                               const int32_t* col_index, int64_t n_new, int64_t zero_rows_from,
                               void* packed_out, void* scales_out, int64_t n_out_pad, int* status_word, void* stream);
int uniql_w4a16_dequantize_rows(const void* packed, const void* scales, int64_t size_k, int64_t n_src_pad,
                                const int32_t* row_index, int64_t k_new, int64_t n_real, void* out, int64_t ld,
                                int* status_word, void* stream);

/*
 * out = silu(gate) * up elementwise on fp16 [rows, cols] (row strides ldg, ldu, ldo; cols and the strides multiples
 * of 8, pointers 16-byte aligned; out may alias gate or up), with the roundings of the separate PyTorch ops (fp16 SiLU,
 * fp16 product).  The part of down_proj(act_fn(gate_proj(x)) * up_proj(x)) (modeling/llama/llama_qblocks.py:48-51) that
 * is left between the launches when the batch has more than 16 rows (up to 16 rows UNIQL_EPILOGUE_SWIGLU does it
 * inside the grouped launch).  One pass instead of two; launched as a programmatic dependent of the launch before it.
 */
int uniql_silu_mul(const void* gate, int64_t ldg, const void* up, int64_t ldu, void* out, int64_t ldo, int64_t rows,
                   int64_t cols, void* stream);

/* Host helper: writes the base x base ±1 matrix (row-major int8) this library uses for
 * base in {12, 20, 28, 40}; `out` is a HOST pointer.  Returns UNIQL_ESHAPE for other orders. */
int uniql_hadamard_base_matrix(int base, int8_t* out);

/* Host call: replaces the order-`base` matrix (12, 20, 28 or 40) used by every transform launched afterwards in this
 * process -- uniql_hadamard, the hadamard_dim argument of the linears, uniql_hadamard_base_matrix.  `h` is a HOST
 * pointer to base*base entries of +1 / -1, row-major, y[a'] = sum_a h[a'*base + a] x[a] on the slow index of
 * i = a * 2^j + b; it is checked for H H^T = base I (UNIQL_EINVAL otherwise).  NULL restores the built-in matrix.
 * The reference takes these matrices from the third-party package fast-hadamard-transform
 * (quantize/hadamard_helpers.py:18-36); a holder of that package's tables passes them here to get its results.
 * Decode-size launches (<= 16 rows) keep their speed; transforms of many rows of a replaced order run on a plainer
 * kernel. */
int uniql_hadamard_set_base_matrix(int base, const int8_t* h);

/*
 * One-shot push all-reduce (sum) of fp16 vectors across the GPUs of one node, for the row-parallel linears of a
 * tensor-parallel model at decode sizes.  No counterpart in the reference (it is single-GPU).  One process per GPU.
 *
 *   uniql_comm_create   allocates this rank's staging block (cudaMalloc, once, at set-up) and writes its CUDA IPC
 *                       handle (uniql_comm_handle_bytes() bytes) to `handle_out` (HOST pointer).  max_elems: largest
 *                       message in fp16 elements (multiple of 8, at most 524288).  The same number sizes the areas the
 *                       decode linear's own exchanges use: read it as 16 batch rows of the widest activation row
 *                       (n <= max_elems / 16 for UNIQL_TP_REDUCE, features <= max_elems / 16 for the gather).
 *   uniql_comm_connect  `all_handles` (HOST pointer) = the handles of ranks 0..world-1 concatenated in rank order
 *                       (exchange them with any host-side channel); opens the peers' blocks.
 *   uniql_allreduce_push  out[i] = sum over ranks of in[i], summed in rank order in fp32, identical on every rank;
 *                       in/out are DEVICE pointers (may alias), count a multiple of 8.  Every rank must issue the same
 *                       sequence of calls.  Peer data is stored into the consumer's memory; waits are bounded
 *                       (UNIQL_STATUS_WAIT_TIMEOUT in *status_word on give-up).  Safe to capture in a CUDA graph.
 */
size_t uniql_comm_handle_bytes(void);
int uniql_comm_create(int rank, int world, int64_t max_elems, void** comm_out, void* handle_out);
int uniql_comm_connect(void* comm, const void* all_handles);
int uniql_comm_destroy(void* comm);
int uniql_allreduce_push(void* comm, const void* in, void* out, int64_t count, int* status_word, void* stream);

/*
 * Row-parallel W4A16 linear with the cross-GPU sum fused into the kernel (decode sizes, m <= 16, n / 64 within the
 * communicator's block capacity max_elems / 1024): D = sum over ranks of (A_rank * dequant(B_rank)) (+ bias), identical
 * on every rank.  The warp that finishes a 64-column block stores its fp16 partial, tagged with an epoch, straight into
 * every rank's staging block over NVLink and then adds up the partials that arrived in its own block (rank order,
 * fp32): the same arithmetic as uniql_w4a16_linear followed by uniql_allreduce_push, in one launch.  No counterpart in
 * the reference.  Staging words are addressed per 64-column block and every block keeps its own epoch, so calls of
 * different shapes may share a communicator; all ranks must issue the same sequence of calls.  Other arguments as for
 * uniql_w4a16_linear (no Hadamard option).
 */
int uniql_w4a16_linear_allreduce(void* comm, const void* A, int64_t lda, const void* B, const void* s,
                                 const void* bias, void* D, int64_t ldd, int64_t m, int64_t n, int64_t n_out,
                                 int64_t k, int groupsize, void* scratch, size_t scratch_bytes, int* status_word,
                                 void* stream);

/*
 * Grouped launch: up to UNIQL_MAX_PROJ projections that read the same activations run as ONE kernel.  For m <= 16 that
 * is the decode kernel with every option below; for 17 <= m <= 128 it is the operand-swapped tensor-core kernel with
 * plain outputs only (epilogue NONE, no residual, no hadamard_dim; every n >= 128) -- q/k/v or gate and up of a block
 * at small batches cost one launch instead of two or three.  Larger m returns UNIQL_ESHAPE.  At decode sizes the
 * elementwise work the reference's blocks do around the projections is folded into the launch.  It replaces
 *   - gate_proj, up_proj and act_fn(gate) * up as three launches (modeling/llama/llama_qblocks.py:48-51):
 *     two projections + UNIQL_EPILOGUE_SWIGLU -> proj[0].D = silu(x W_gate + b_gate) * (x W_up + b_up), with the same
 *     fp16 roundings as the separate modules (proj[1].D is not written); both projections must have the same n, n_out;
 *   - q_proj, k_proj, v_proj as three launches (:104-106): three projections, UNIQL_EPILOGUE_NONE, each writing its own D;
 *   - the residual add after o_proj / down_proj: `residual` (fp16 [m, n_out], row stride ldr, may alias D) is added to
 *     the rounded result (single projection or SwiGLU pair);
 *   - the Hadamard module in front of down_proj / out_proj (quantize/quant_hadamard_layers.py:16-18): hadamard_dim = k
 *     transforms every activation row first (rounded to fp16 as the module would): a few-row kernel in front whose
 *     launch the linear's weight stream overlaps (in the slot-balanced kernel's own prologue for m <= 4).
 * Each projection is described by plain pointers and sizes (see uniql_w4a16_linear for B, s, bias, D, n, n_out).
 * scratch: at least uniql_w4a16_group_scratch_bytes(...) bytes, 256-byte aligned, first UNIQL_SCRATCH_COUNTER_BYTES
 * zero before the first call (every call leaves them zero).  The weights and scales must not be written by the kernel
 * that immediately precedes this call in the stream (the launch starts fetching them before that kernel has ended);
 * activations, bias, residual and outputs have no such restriction.
 */
#define UNIQL_MAX_PROJ 4
enum { UNIQL_EPILOGUE_NONE = 0, UNIQL_EPILOGUE_SWIGLU = 1 };
typedef struct uniql_w4a16_proj {
  const void* B;       /* int32 [k/16, 2*n] */
  const void* s;       /* fp16 [k/128, n] */
  const void* bias;    /* fp16 [n_out] or NULL */
  void* D;             /* fp16 [m, n_out], row stride ldd */
  int64_t ldd;
  int64_t n, n_out;
} uniql_w4a16_proj;
/* Optional hint: byte ranges (at most UNIQL_MAX_PREFETCH, 128-byte aligned device pointers) that the launch asks L2
 * for as soon as its own weight stream ends -- the packed weights of the launches that come next in the decode step.
 * HBM then keeps working while this launch drains and the next one starts.  Pure hint: no effect on results. */
#define UNIQL_MAX_PREFETCH 4
typedef struct uniql_prefetch {
  const void* ptr;
  size_t bytes;
} uniql_prefetch;
int uniql_w4a16_linear_group(const void* A, int64_t lda, int64_t m, int64_t k, const uniql_w4a16_proj* proj,
                             int nproj, int epilogue, const void* residual, int64_t ldr, int64_t hadamard_dim,
                             const uniql_prefetch* next, int nnext, void* scratch, size_t scratch_bytes,
                             int* status_word, void* stream);
size_t uniql_w4a16_group_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue,
                                       int64_t hadamard_dim);

/*
 * The same launch as one step of a tensor-parallel layer (one process per GPU, `comm` from uniql_comm_create /
 * uniql_comm_connect).  No counterpart in the reference.  `flags` selects what crosses NVLink, always as epoch-tagged
 * 8-byte words stored into the consumer's memory, every wait bounded (UNIQL_STATUS_WAIT_TIMEOUT on give-up):
 *   UNIQL_TP_REDUCE      row-parallel shard: the result is summed over the ranks inside the kernel (as
 *                        uniql_w4a16_linear_allreduce; bias and residual are added once, after the sum).
 *   UNIQL_TP_GATHER_OUT  column-parallel shard (one projection or a SwiGLU pair, n_out even): besides D, the result
 *                        columns are stored at feature index col_offset + column into every rank's feature area.
 *   UNIQL_TP_GATHER_IN   the activations are the full row assembled in this rank's feature area by the preceding
 *                        UNIQL_TP_GATHER_OUT launches of all ranks (A is ignored); requires hadamard_dim (the size of
 *                        the full row, at most max_elems / 16) with k_offset = first feature of this rank's k range:
 *                        every rank transforms the row and keeps its own slice.  Call it directly after the
 *                        GATHER_OUT launch it pairs with, and follow it by a UNIQL_TP_REDUCE (usually the same call).
 */
enum { UNIQL_TP_REDUCE = 1, UNIQL_TP_GATHER_OUT = 2, UNIQL_TP_GATHER_IN = 4 };
int uniql_w4a16_linear_group_tp(void* comm, int flags, int64_t col_offset, int64_t k_offset, const void* A,
                                int64_t lda, int64_t m, int64_t k, const uniql_w4a16_proj* proj, int nproj,
                                int epilogue, const void* residual, int64_t ldr, int64_t hadamard_dim,
                                const uniql_prefetch* next, int nnext, void* scratch, size_t scratch_bytes,
                                int* status_word, void* stream);

/*
 * Host-only check of the decode kernel's work split for one launch geometry (no GPU work is enqueued): replays every
 * warp's slot range with the kernel's own index arithmetic and verifies that each (block, group) slot is streamed
 * exactly once, that every partial tile has its own place in scratch and that the per-block tickets add up.
 * Returns 0, a negative UNIQL_E* code for a geometry the kernel does not take, or a positive number naming the
 * check that failed.  *fused_hadamard_out (may be NULL) tells whether the Hadamard would run in the kernel prologue.
 */
int uniql_w4a16_plan_selftest(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t hadamard_dim,
                              int64_t k_offset, int* fused_hadamard_out);

/* Host-only check of the plan the CTA-tiled decode kernel would use for a launch of this shape (no device work, usable
 * without a GPU): the invariants its index arithmetic relies on (warp arrangement, split, shared-memory carve-up, scratch
 * size) and that the k-ranges of its warps cover every packed row exactly once.  Returns 0, or the number of the check
 * that failed; out5 (may be NULL) receives {WN, S, cluster (0/1), dynamic shared memory bytes, partial-sum bytes}. */
int uniql_w4a16_gemv_plan_check(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t* out5);

#ifdef __cplusplus
}
#endif
#endif /* UNIQL_B200_H_ */
