// Load-time slicing primitives for packed W4A16 layers on sm_100a.
//
// UniQL re-slices its packed weights at every load of an elastic checkpoint
// (modeling/modeling_helpers.py:235-867: slice_w4a16_{up_gate,down,qk,v,o,in,out}_proj) by unpacking to one int per
// weight on the CPU, slicing and packing again (quantize/quantize_helpers.py:279-328, :67-84).  The two kernels here do
// the same work directly on the packed buffers:
//   * w4a16_gather_columns_kernel: new layer = chosen output columns of an old one (q/k/v/in_proj slicing).  An output
//     word holds 4 k-values x 2 columns; the 4 nibbles of one column sit in ONE source word (same packed row, same k
//     sub-position), so an output word is assembled from two source words and a few shifts.  Scales are gathered
//     through the 64-column scale permutation.
//   * w4a16_dequantize_rows_kernel: fp16 (q - 8) * s of chosen input rows, written in the nn.Linear layout
//     [column][kept row] that uniql_w4a16_quantize reads (o_proj / out_proj slicing re-quantises, :632-650).
// Both are gathers of 4-byte words: memory-bound, run once per layer at load time.
#include "common.cuh"

namespace uniql {

namespace {

// position of column r (0..63) of a 64-column block inside a packed row, and its scale slot
struct ColPos {
  int j, g, hi;       // register index, fragment row, +8 half
};
__device__ __forceinline__ ColPos col_pos(int r) {
  ColPos p;
  p.j = r >> 4;
  p.g = r & 7;
  p.hi = (r >> 3) & 1;
  return p;
}
__device__ __forceinline__ int scale_slot(int r) { return 8 * (r & 7) + (r >> 3); }   // stored[8 i + j] = natural[i + 8 j]

__global__ void __launch_bounds__(128)
w4a16_gather_columns_kernel(const uint32_t* __restrict__ packed_in, const __half* __restrict__ scales_in, int n_src_pad,
                            const int* __restrict__ col_index, int n_new, int zero_rows_from,
                            uint32_t* __restrict__ packed_out, __half* __restrict__ scales_out, int n_out_pad,
                            int* __restrict__ status_word) {
  const int w = threadIdx.x;                     // output word of this 64-column block and packed row
  const int b = blockIdx.x, kt = blockIdx.y;
  const int i = w >> 2, j = w & 3, g = i >> 2, c = i & 3;
  uint32_t out = 0;
#pragma unroll
  for (int hi = 0; hi < 2; ++hi) {
    const int n_out = 64 * b + 16 * j + g + 8 * hi;
    int src = n_out < n_new ? col_index[n_out] : -1;
    if (src >= n_src_pad) {                      // not a column of the source: zero column, and say so
      if (status_word) atomicOr(status_word, UNIQL_STATUS_BAD_INDEX);
      src = -1;
    }
    if (src < 0) continue;
    const ColPos sp = col_pos(src & 63);
    const uint32_t word = packed_in[(size_t)kt * (2 * (size_t)n_src_pad) + (size_t)(src >> 6) * 128 + (sp.g * 4 + c) * 4 + sp.j];
#pragma unroll
    for (int bit1 = 0; bit1 < 2; ++bit1)
#pragma unroll
      for (int bit8 = 0; bit8 < 2; ++bit8) {
        const int k = 16 * kt + 2 * c + bit1 + 8 * bit8;
        if (k >= zero_rows_from) continue;
        const uint32_t q = (word >> (4 * (bit8 + 2 * sp.hi + 4 * bit1))) & 0xFu;
        out |= q << (4 * (bit8 + 2 * hi + 4 * bit1));
      }
  }
  packed_out[(size_t)kt * (2 * (size_t)n_out_pad) + (size_t)b * 128 + w] = out;

  if ((kt & 7) == 0 && w < 64) {                 // one scale row per 8 packed rows
    const int grp = kt >> 3;
    const int r = (w >> 3) + 8 * (w & 7);        // natural column stored at slot w
    const int n_out = 64 * b + r;
    const int src = n_out < n_new ? col_index[n_out] : -1;
    __half s = __float2half(0.f);
    if (src >= 0 && src < n_src_pad) s = scales_in[(size_t)grp * n_src_pad + (size_t)(src >> 6) * 64 + scale_slot(src & 63)];
    scales_out[(size_t)grp * n_out_pad + 64 * b + w] = s;
  }
}

__global__ void __launch_bounds__(256)
w4a16_dequantize_rows_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scales, int size_k,
                             int n_src_pad, const int* __restrict__ row_index, int k_new, int n_real,
                             __half* __restrict__ out, int64_t ld, int* __restrict__ status_word) {
  // consecutive threads take consecutive kept rows of one column: coalesced writes, gathered 4-byte reads
  const int kk = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (kk >= k_new || n >= n_real) return;
  const int k = row_index[kk];
  if (k < 0 || k >= size_k) {                    // not a row of the source: zero, and say so
    if (status_word) atomicOr(status_word, UNIQL_STATUS_BAD_INDEX);
    out[(size_t)n * ld + kk] = __float2half(0.f);
    return;
  }
  const int kt = k >> 4, k16 = k & 15;
  const int c = (k16 & 7) >> 1, bit1 = k16 & 1, bit8 = k16 >> 3;
  const ColPos p = col_pos(n & 63);
  const uint32_t word = packed[(size_t)kt * (2 * (size_t)n_src_pad) + (size_t)(n >> 6) * 128 + (p.g * 4 + c) * 4 + p.j];
  const int q = (int)((word >> (4 * (bit8 + 2 * p.hi + 4 * bit1))) & 0xFu);
  const __half s = scales[(size_t)(k >> 7) * n_src_pad + (size_t)(n >> 6) * 64 + scale_slot(n & 63)];
  // (q - 8) is exact in fp16; one rounding of the product, as the fp16 tensor multiply of the reference
  out[(size_t)n * ld + kk] = __hmul(__int2half_rn(q - 8), s);
}

}  // namespace

}  // namespace uniql

extern "C" int uniql_w4a16_gather_columns(const void* packed_in, const void* scales_in, int64_t size_k, int64_t n_src_pad,
                                          const int32_t* col_index, int64_t n_new, int64_t zero_rows_from,
                                          void* packed_out, void* scales_out, int64_t n_out_pad, int* status_word,
                                          void* stream) {
  using namespace uniql;
  if (size_k <= 0 || size_k % 128 != 0 || n_src_pad <= 0 || n_src_pad % 64 != 0) return UNIQL_ESHAPE;
  if (n_out_pad <= 0 || n_out_pad % 64 != 0 || n_new < 0 || n_new > n_out_pad) return UNIQL_ESHAPE;
  if (size_k / 16 > 65535) return UNIQL_ESHAPE;
  if (!packed_in || !scales_in || !packed_out || !scales_out || (n_new > 0 && !col_index)) return UNIQL_EINVAL;
  if (zero_rows_from < 0 || zero_rows_from > size_k) zero_rows_from = size_k;
  dim3 grid((unsigned)(n_out_pad / 64), (unsigned)(size_k / 16));
  w4a16_gather_columns_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)packed_in, (const __half*)scales_in, (int)n_src_pad, col_index, (int)n_new, (int)zero_rows_from,
      (uint32_t*)packed_out, (__half*)scales_out, (int)n_out_pad, status_word);
  return launch_status();
}

extern "C" int uniql_w4a16_dequantize_rows(const void* packed, const void* scales, int64_t size_k, int64_t n_src_pad,
                                           const int32_t* row_index, int64_t k_new, int64_t n_real, void* out, int64_t ld,
                                           int* status_word, void* stream) {
  using namespace uniql;
  if (size_k <= 0 || size_k % 128 != 0 || n_src_pad <= 0 || n_src_pad % 64 != 0) return UNIQL_ESHAPE;
  if (k_new < 0 || n_real < 0 || n_real > n_src_pad || n_real > 65535 || ld < k_new) return UNIQL_ESHAPE;
  if (k_new == 0 || n_real == 0) return UNIQL_OK;
  if (!packed || !scales || !row_index || !out) return UNIQL_EINVAL;
  dim3 grid((unsigned)((k_new + 255) / 256), (unsigned)n_real);
  w4a16_dequantize_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)packed, (const __half*)scales, (int)size_k, (int)n_src_pad, row_index, (int)k_new, (int)n_real,
      (__half*)out, ld, status_word);
  return launch_status();
}
