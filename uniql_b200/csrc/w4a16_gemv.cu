// Decode-regime W4A16 linear (m <= 16) for sm_100a: a weight-streaming skinny GEMM.
//
// Replaces the small-batch instantiations of UniQL's Marlin kernel
// (csrc/linear/marlin_gemm_kernel.cuh:176-740, tile table :792-800) while consuming the very same
// packed buffers (quantize/quantize_helpers.py:145-165 weight order, :54-62 scale order).
//
// How the packed layout is consumed.  Packed row kt (16 k-values) holds, for every 64-column block,
// 512 contiguous bytes; lane i of a warp owns bytes 16i..16i+15 = four words j=0..3.  With g = i/4 and
// c = i%4, word j carries W[k, n] for k = 16kt + {2c, 2c+1, 2c+8, 2c+9} and n = 64blk + 16j + g + {0, 8}.
// That is exactly the A-operand fragment of mma.m16n8k16 when the *weights* are the 16-row operand
// (rows = 16 output columns) and the activations are the 8-column operand (columns = batch rows).
// So one 16-byte load per lane feeds four tensor-core instructions per 8 batch rows with no data
// movement between lanes, and all 16 rows of the MMA do useful work even at m = 1.
//
// Parallelisation.  A CTA has 8 warps arranged WN (along n, adjacent 64-column blocks) x WK (along k).
// The grid is (ceil(n/64/WN), S): S CTAs split k.  Every warp streams its own contiguous k-range with
// a ring of 8 outstanding 16-byte loads per lane (one quantisation group ahead), L2 evict-first.
// Group scales are applied to the fp32 group accumulator once per group (16 FMAs) instead of once per
// weight.  Warps of a CTA are reduced through shared memory in a fixed order; CTAs along k write fp32
// partials to scratch and the last one to arrive (atomic ticket, no spinning) adds them in a fixed
// order -> deterministic results, no inter-CTA waits.
//
// Roofline: HBM.  Algorithmic bytes per launch = k*n/2 + (k/128)*n*2 + m*k*2 + m*n_out*2.
#include "common.cuh"
#include "linear_internal.cuh"

#include <stdlib.h>

namespace uniql {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;
constexpr int kRedStride = 68;  // floats per row of a warp's 64-column reduction tile (+4: conflict-free scatter)

struct GemvParams {
  const __half* A;
  int64_t lda;
  const uint4* B;       // packed weights, row kt has n/2 uint4
  const uint4* S;       // permuted scales, row g has n/8 uint4
  const __half* bias;
  __half* D;
  int64_t ldd;
  int M, N, n_out, KT, nblk;
  int WN, WK, S_split, GCH;
  int xs_stride;        // halves per staged activation row (GCH*128 + 8)
  float* partials;      // [S_split][M][N]
  int* counters;        // [gridDim.x], zero on entry, zero on exit
  int pdl;              // 1: launched as a programmatic dependent of the kernel that produces A
};

template <int MT>
__global__ void __launch_bounds__(kGemvThreads, 2) w4a16_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ int s_is_last;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int wn = warp % p.WN, wk = warp / p.WN;
  const int blk = blockIdx.x * p.WN + wn;
  const bool active = blk < p.nblk;

  // k-range of this CTA, then of this warp row (contiguous, balanced to one packed row).
  const int cta_k0 = (int)((int64_t)p.KT * blockIdx.y / p.S_split);
  const int cta_k1 = (int)((int64_t)p.KT * (blockIdx.y + 1) / p.S_split);
  const int w0 = cta_k0 + (int)((int64_t)(cta_k1 - cta_k0) * wk / p.WK);
  const int w1 = cta_k0 + (int)((int64_t)(cta_k1 - cta_k0) * (wk + 1) / p.WK);
  const int g0 = w0 >> 3, g1 = (w1 + 7) >> 3;   // quantisation groups touched (8 packed rows each)

  const uint64_t pol = make_evict_first_policy();
  const int64_t row_u4 = p.N >> 1;                          // uint4 per packed row
  const uint4* wptr = p.B + (int64_t)blk * 32 + lane;       // + kt * row_u4
  const uint4* sptr = p.S + (int64_t)blk * 8 + g;           // + grp * (N/8)
  const int64_t srow_u4 = p.N >> 3;

  // ---- fill the ring before anything else so HBM requests are in flight while x is staged ----
  uint4 ring[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int kt = 8 * g0 + u;
    ring[u] = make_uint4(0, 0, 0, 0);
    if (active && kt >= w0 && kt < w1) ring[u] = ld_stream16(wptr + (int64_t)kt * row_u4, pol);
  }
  uint4 s_cur = make_uint4(0, 0, 0, 0);
  if (active && g0 < g1) s_cur = ld_nc16(sptr + (int64_t)g0 * srow_u4);

  if (p.pdl) pdl_wait();   // activations may come from the preceding kernel

  __half* xs = reinterpret_cast<__half*>(smem_raw) + (size_t)wk * (8 * MT) * p.xs_stride;
  const int row_threads = p.WN * 32;
  const int row_tid = wn * 32 + lane;

  float acc[MT][4][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[t][j][r] = 0.f;

  for (int gi = g0; gi < g1; ++gi) {
    // ---- stage the next chunk of activations for this warp row (GCH groups = GCH*128 k-values) ----
    if ((gi - g0) % p.GCH == 0) {
      asm volatile("bar.sync %0, %1;" ::"r"(wk + 1), "r"(row_threads));
      const int gend = min(gi + p.GCH, g1);
      const int vec_per_row = (gend - gi) * 16;               // 16-byte vectors per row
      const int total = 8 * MT * vec_per_row;
      for (int v = row_tid; v < total; v += row_threads) {
        const int r = v / vec_per_row, col = v - r * vec_per_row;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < p.M) val = ld_nc16(p.A + (int64_t)r * p.lda + (int64_t)gi * 128 + col * 8);
        *reinterpret_cast<uint4*>(xs + (size_t)r * p.xs_stride + col * 8) = val;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(wk + 1), "r"(row_threads));
    }
    uint4 s_next = make_uint4(0, 0, 0, 0);
    if (active && gi + 1 < g1) s_next = ld_nc16(sptr + (int64_t)(gi + 1) * srow_u4);

    float accg[MT][4][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) accg[t][j][r] = 0.f;

    const __half* xg = xs + (size_t)((gi - g0) % p.GCH) * 128;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int kt = 8 * gi + u;
      const uint4 cur = ring[u];
      if (active && kt + 8 < w1) ring[u] = ld_stream16(wptr + (int64_t)(kt + 8) * row_u4, pol);
      if (active && kt >= w0 && kt < w1) {
        uint32_t b0[MT], b1[MT];
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const __half* xr = xg + (size_t)(8 * t + g) * p.xs_stride + u * 16 + 2 * c;
          b0[t] = *reinterpret_cast<const uint32_t*>(xr);
          b1[t] = *reinterpret_cast<const uint32_t*>(xr + 8);
        }
        const uint32_t wq[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a[4];
          const uint32_t q = wq[j], qs = wq[j] >> 8;
          a[0] = nib_pair_to_half2_m8(q);        // n = 16j+g,   k = 2c, 2c+1
          a[2] = nib_pair_hi_to_half2_m8(q);     // n = 16j+g,   k = 2c+8, 2c+9
          a[1] = nib_pair_to_half2_m8(qs);       // n = 16j+g+8, k = 2c, 2c+1
          a[3] = nib_pair_hi_to_half2_m8(qs);    // n = 16j+g+8, k = 2c+8, 2c+9
#pragma unroll
          for (int t = 0; t < MT; ++t) mma_m16n8k16(accg[t][j], a, b0[t], b1[t]);
        }
      }
    }
    // ---- apply this group's scales: lane holds s[64blk + 8g + 2j + b] for j=0..3, b=0..1 ----
    {
      const __half2* sh = reinterpret_cast<const __half2*>(&s_cur);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 sf = __half22float2(sh[j]);   // .x -> columns 16j+g, .y -> 16j+g+8
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          acc[t][j][0] = fmaf(accg[t][j][0], sf.x, acc[t][j][0]);
          acc[t][j][1] = fmaf(accg[t][j][1], sf.x, acc[t][j][1]);
          acc[t][j][2] = fmaf(accg[t][j][2], sf.y, acc[t][j][2]);
          acc[t][j][3] = fmaf(accg[t][j][3], sf.y, acc[t][j][3]);
        }
      }
    }
    s_cur = s_next;
  }

  // ---- reduce the WK warp rows through shared memory (fixed order) ----
  __syncthreads();   // everyone is done with the staged activations; reuse the space
  float* red = reinterpret_cast<float*>(smem_raw);
  {
    float* mine = red + (size_t)warp * (8 * MT) * kRedStride;
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int m = 8 * t + 2 * c + (r & 1);
          const int nl = 16 * j + g + 8 * (r >> 1);
          mine[m * kRedStride + nl] = acc[t][j][r];
        }
  }
  __syncthreads();

  const int cta_cols = p.WN * 64;
  const int n_base = blockIdx.x * cta_cols;
  const int total = p.M * cta_cols;
  const bool direct = (p.S_split == 1);
  for (int idx = tid; idx < total; idx += kGemvThreads) {
    const int m = idx / cta_cols, col = idx - m * cta_cols;
    const int n = n_base + col;
    if (n >= p.N) continue;
    const int wn_i = col >> 6, nl = col & 63;
    float v = 0.f;
    for (int k = 0; k < p.WK; ++k) v += red[((size_t)(k * p.WN + wn_i) * (8 * MT) + m) * kRedStride + nl];
    if (direct) {
      if (n < p.n_out) {
        if (p.bias) v += __half2float(p.bias[n]);
        p.D[(int64_t)m * p.ldd + n] = __float2half_rn(v);
      }
    } else {
      p.partials[((size_t)blockIdx.y * p.M + m) * p.N + n] = v;
    }
  }
  if (direct) return;

  // ---- split-k: the last CTA of this column group to finish adds the partials ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(p.counters + blockIdx.x, 1);
    const int last = (ticket == p.S_split - 1);
    if (last) p.counters[blockIdx.x] = 0;   // leave the counter clean for the next launch
    s_is_last = last;
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();
  for (int idx = tid; idx < total; idx += kGemvThreads) {
    const int m = idx / cta_cols, col = idx - m * cta_cols;
    const int n = n_base + col;
    if (n >= p.n_out) continue;
    float v = 0.f;
    for (int s = 0; s < p.S_split; ++s) v += __ldcg(p.partials + ((size_t)s * p.M + m) * p.N + n);
    if (p.bias) v += __half2float(p.bias[n]);
    p.D[(int64_t)m * p.ldd + n] = __float2half_rn(v);
  }
}

// ------------------------------------------------------------------ host side
static int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

GemvPlan plan_gemv(int64_t m, int64_t n, int64_t k) {
  GemvPlan best{};
  const int nblk = (int)(n / 64), KT = (int)(k / 16);
  const int slots = device_info().sm_count * 2;
  double best_cost = 1e30;
  for (int WN = 8; WN >= 1; WN >>= 1) {
    const int WK = kGemvWarps / WN;
    const int groups = (nblk + WN - 1) / WN;
    const double waste = (double)(groups * WN) / nblk;   // idle warps in the last column group
    const int smax = KT / WK < 1 ? 1 : (KT / WK > 64 ? 64 : KT / WK);
    for (int S = 1; S <= smax; ++S) {
      const int64_t ctas = (int64_t)groups * S;
      const int64_t waves = (ctas + slots - 1) / slots;
      const int per_cta = (KT + S - 1) / S;
      const int len = (per_cta + WK - 1) / WK;           // packed rows streamed by one warp
      // cost in "packed rows per warp": streamed rows + fixed latency per wave + split-k reduction
      double cost = (double)waves * (len + 10.0) * waste + (S > 1 ? 3.0 + 0.35 * S : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best.WN = WN; best.WK = WK; best.S = S;
      }
    }
  }
  const int ov_wn = env_int("UNIQL_B200_GEMV_WN", 0), ov_s = env_int("UNIQL_B200_GEMV_S", 0);
  if (ov_wn == 1 || ov_wn == 2 || ov_wn == 4 || ov_wn == 8) { best.WN = ov_wn; best.WK = kGemvWarps / ov_wn; }
  if (ov_s >= 1) best.S = ov_s;
  if (best.S > KT) best.S = KT;
  const int MT = m <= 8 ? 1 : 2;
  // activation staging: WK warp rows x 8*MT batch rows x (GCH*128 + 8) halves, kept under ~40 KB
  int gch = (int)((40960 / (best.WK * 8 * MT * 2) - 8) / 128);
  if (gch < 1) gch = 1;
  if (gch > 8) gch = 8;
  best.GCH = gch;
  best.MT = MT;
  const size_t xs_bytes = (size_t)best.WK * 8 * MT * (gch * 128 + 8) * 2;
  const size_t red_bytes = (size_t)kGemvWarps * 8 * MT * kRedStride * 4;
  best.smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  best.partial_bytes = best.S > 1 ? (size_t)best.S * (size_t)(m < 16 ? m : 16) * n * 4 : 0;
  return best;
}

static inline int grid_x_of(const GemvParams& p) { return (p.nblk + p.WN - 1) / p.WN; }

int launch_gemv(const LinearArgs& a, const __half* A, int64_t lda, __half* D, int64_t m, const GemvPlan& plan,
                bool pdl, cudaStream_t stream) {
  GemvParams p;
  p.A = A; p.lda = lda;
  p.B = (const uint4*)a.B; p.S = (const uint4*)a.s; p.bias = (const __half*)a.bias;
  p.D = D; p.ldd = a.ldd;
  p.M = (int)m; p.N = (int)a.n; p.n_out = (int)a.n_out; p.KT = (int)(a.k / 16); p.nblk = (int)(a.n / 64);
  p.WN = plan.WN; p.WK = plan.WK; p.S_split = plan.S; p.GCH = plan.GCH;
  p.xs_stride = plan.GCH * 128 + 8;
  p.counters = a.counters;
  p.partials = a.partials;
  if (plan.partial_bytes > a.partial_bytes) return UNIQL_ESCRATCH;
  if ((size_t)grid_x_of(p) * sizeof(int) > UNIQL_SCRATCH_COUNTER_BYTES) return UNIQL_ESHAPE;
  p.pdl = pdl ? 1 : 0;
  dim3 grid(grid_x_of(p), p.S_split);

  auto kern = plan.MT == 1 ? w4a16_gemv_kernel<1> : w4a16_gemv_kernel<2>;
  static thread_local bool attr_set[2] = {false, false};
  if (plan.smem > 48 * 1024 && !attr_set[plan.MT - 1]) {
    UNIQL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    attr_set[plan.MT - 1] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  UNIQL_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return UNIQL_OK;
}

}  // namespace uniql
