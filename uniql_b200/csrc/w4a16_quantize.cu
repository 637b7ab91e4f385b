// Round-to-nearest group-128 int4 quantiser + packer for sm_100a: fp16 nn.Linear weight [N, K] -> the packed
// buffers the linear kernels consume, in one pass over the weight.
//
// Replaces the CPU path of W4A16B16O16Linear.from_fp16 (quantize/quant_linear_layers.py:50-89), i.e.
// w4a16_quantize(W^T, 4, 128, scale, pad_out) (quantize/quantize_helpers.py:184-241): RTN of
// get_fake_quantize_weights (:88-141: per group of 128 k and column n, s = max|w| * 2/15 in fp16,
// q = clamp(round(w / s) + 8, 0, 15), w_ref = (q - 8) * s), the code path for scales handed in by GPTQ (:205-218), the
// Marlin weight order (:145-165, :38-50, :67-84) and the scale order (:54-62, :169-180).  Every intermediate is rounded
// to fp16 where torch's fp16 CPU kernels round, so packed words, scales and w_ref are bit-identical to the reference.
//
// One CTA per (64-column block, group): the 64 x 128 tile is read with 16-byte coalesced loads from the [N, K]
// layout (no transposed copy on the host), reduced to per-column scales, quantised, and written as 8 packed rows of 128
// words (512 contiguous bytes each).  Bound: HBM; 2 bytes read and 0.5 written per weight (+2 with w_ref).
#include "common.cuh"

namespace uniql {

namespace {

constexpr int kQThreads = 256;
constexpr int kTileN = 64, kTileK = 128;
constexpr int kTilePad = 8;    // halves of padding per tile row

struct QuantParams {
  const __half* W;          // [n_out, k_in], row stride ldw
  int64_t ldw;
  int n_out, k_in;
  const __half* gscale;     // optional [groups, n_out], natural column order
  uint32_t* packed;         // [Kp/16, 2 * n_pad]
  __half* scales;           // [Kp/128, n_pad], permuted inside 64-column blocks
  __half* w_ref;            // optional [Kp, n_pad]
  int n_pad;
};

template <bool HAS_SCALE>
__global__ void __launch_bounds__(kQThreads)
w4a16_quantize_kernel(const QuantParams p) {
  __shared__ __align__(16) __half wref[kTileK][kTileN + kTilePad];   // [k][column], only filled when w_ref is wanted
  __shared__ uint8_t codes[kTileK][kTileN + 4];
  __shared__ __half col_scale[kTileN];

  const int t = threadIdx.x;
  const int n0 = blockIdx.x * kTileN, k0 = blockIdx.y * kTileK;

  // ---- load: 16 lanes per weight row (= output column), 8 consecutive k each, 16 columns per pass; the four passes'
  //      loads are issued together and the values stay in registers.  Rows / k past the matrix read as zero. ----
  const bool vec_ok = ((p.ldw & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.W) & 15u) == 0);
  const int r = t >> 4, seg = t & 15;
  constexpr int kPasses = kTileN / 16;
  uint4 raw[kPasses];
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int gn = n0 + pass * 16 + r, gk = k0 + seg * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gn < p.n_out) {
      const __half* src = p.W + (size_t)gn * p.ldw + gk;
      if (vec_ok && gk + 8 <= p.k_in) {
        v = *reinterpret_cast<const uint4*>(src);
      } else {
        __half h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = (gk + e < p.k_in) ? src[e] : __float2half(0.f);
        v = *reinterpret_cast<uint4*>(h);
      }
    }
    raw[pass] = v;
  }

#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int n = pass * 16 + r;
    const bool real_col = n0 + n < p.n_out;
    const __half* h8 = reinterpret_cast<const __half*>(&raw[pass]);
    __half s16;
    if (HAS_SCALE) {
      s16 = real_col ? p.gscale[(size_t)blockIdx.y * p.n_out + n0 + n] : __float2half(0.f);
    } else {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(__half2float(h8[e])));
      // the 16 lanes of a column are one half of the warp: xor steps 1..8 stay inside it
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
      // fp16 tensor times the Python scalar 2/15: one fp32 multiply, one rounding to fp16
      s16 = __float2half_rn(__fmul_rn(amax, (float)(2.0 / 15.0)));
    }
    if (seg == 0) col_scale[n] = s16;
    const float s = __half2float(s16);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int k = seg * 8 + e;
      const __half w16 = h8[e];
      const float w = __half2float(w16);
      int q;
      __half ref;
      if (!real_col) {                              // padded output column: zero code, zero scale, +0 reference
        q = 0;
        ref = __float2half(0.f);
      } else if (HAS_SCALE) {
        // the weight is already on the grid of the given scales: q = round(fp16(fp16(w / s) + 8)), NaN and inf -> 0
        const __half ratio = __float2half_rn(__fdiv_rn(w, s));
        const float shifted = __half2float(__float2half_rn(__fadd_rn(__half2float(ratio), 8.f)));
        q = (isnan(shifted) || isinf(shifted)) ? 0 : (int)rintf(shifted);
        q = min(max(q, 0), 15);
        ref = w16;
      } else {
        // q = clamp(round(fp16(w / s)) + 8, 0, 15); an all-zero group (s = 0, w / s = NaN) gets code 0
        const __half ratio = __float2half_rn(__fdiv_rn(w, s));
        const float rf = __half2float(ratio);
        q = (s == 0.f || isnan(rf)) ? 0 : min(max((int)rintf(rf) + 8, 0), 15);
        ref = __float2half_rn(__fmul_rn((float)(q - 8), s));
      }
      codes[k][n] = (uint8_t)q;
      if (p.w_ref) wref[k][n] = ref;
    }
  }
  __syncthreads();

  // ---- pack: word w of packed row kt belongs to lane i = w / 4 (g = i / 4, c = i % 4), register j = w % 4, and
  //      holds, from the low nibble up, (k, n) = (2c, g) (2c+8, g) (2c, g+8) (2c+8, g+8) (2c+1, g) (2c+9, g)
  //      (2c+1, g+8) (2c+9, g+8) with k relative to 16 kt and n relative to 16 j ----
  {
    const int w = t & 127;
    const int i = w >> 2, j = w & 3, g = i >> 2, c = i & 3;
    const int col = 16 * j + g;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int kt = pass * 2 + (t >> 7);
      const int kb = 16 * kt + 2 * c;
      const uint32_t word = (uint32_t)codes[kb][col] | ((uint32_t)codes[kb + 8][col] << 4) |
                            ((uint32_t)codes[kb][col + 8] << 8) | ((uint32_t)codes[kb + 8][col + 8] << 12) |
                            ((uint32_t)codes[kb + 1][col] << 16) | ((uint32_t)codes[kb + 9][col] << 20) |
                            ((uint32_t)codes[kb + 1][col + 8] << 24) | ((uint32_t)codes[kb + 9][col + 8] << 28);
      p.packed[((size_t)blockIdx.y * 8 + kt) * (2 * (size_t)p.n_pad) + (size_t)blockIdx.x * 128 + w] = word;
    }
  }
  // ---- scales, permuted inside the block: stored[8 i + j] = natural[i + 8 j] ----
  if (t < kTileN) p.scales[(size_t)blockIdx.y * p.n_pad + n0 + t] = col_scale[(t >> 3) + 8 * (t & 7)];
  // ---- reference weights, [k][n] rows of 64 halves ----
  if (p.w_ref) {
    const int k = t >> 1, h0 = (t & 1) * 32;
    __half* dst = p.w_ref + (size_t)(k0 + k) * p.n_pad + n0 + h0;
    if ((p.n_pad & 7) == 0 && (reinterpret_cast<uintptr_t>(p.w_ref) & 15u) == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
        *reinterpret_cast<uint4*>(dst + 8 * v) = *reinterpret_cast<const uint4*>(&wref[k][h0 + 8 * v]);
    } else {
      for (int e = 0; e < 32; ++e) dst[e] = wref[k][h0 + e];
    }
  }
}

}  // namespace

}  // namespace uniql

extern "C" int uniql_w4a16_quantize(const void* W, int64_t ldw, int64_t n_out, int64_t k_in, const void* group_scale,
                                    void* packed, void* scales, void* w_ref, int64_t n_pad, void* stream_) {
  using namespace uniql;
  if (n_out <= 0 || k_in <= 0 || ldw < k_in) return UNIQL_EINVAL;
  if (n_pad < n_out || n_pad % 64 != 0) return UNIQL_ESHAPE;
  if (n_pad > ((int64_t)1 << 22) || k_in > ((int64_t)1 << 22)) return UNIQL_ESHAPE;
  if (!W || !packed || !scales) return UNIQL_EINVAL;
  if ((reinterpret_cast<uintptr_t>(W) & 1u) || (reinterpret_cast<uintptr_t>(packed) & 3u) ||
      (reinterpret_cast<uintptr_t>(scales) & 1u) || (reinterpret_cast<uintptr_t>(w_ref) & 1u) ||
      (reinterpret_cast<uintptr_t>(group_scale) & 1u))
    return UNIQL_EINVAL;
  QuantParams p;
  p.W = (const __half*)W; p.ldw = ldw; p.n_out = (int)n_out; p.k_in = (int)k_in;
  p.gscale = (const __half*)group_scale;
  p.packed = (uint32_t*)packed; p.scales = (__half*)scales; p.w_ref = (__half*)w_ref; p.n_pad = (int)n_pad;
  const int64_t groups = (k_in + 127) / 128;
  if (groups > 65535) return UNIQL_ESHAPE;
  dim3 grid((unsigned)(n_pad / 64), (unsigned)groups);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (group_scale) w4a16_quantize_kernel<true><<<grid, kQThreads, 0, stream>>>(p);
  else w4a16_quantize_kernel<false><<<grid, kQThreads, 0, stream>>>(p);
  return launch_status();
}
