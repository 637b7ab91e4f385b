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
// The grid is (ceil(blocks/WN), S): S CTAs split k.  Every warp streams its own contiguous k-range through a ring of
// two or three 4 KB shared-memory slots that one elected lane fills with 2-D TMA tiles (one quantisation group of one
// 64-column block each, L2 evict-first, no multicast; bounded mbarrier waits).  Group scales are applied to the fp32
// group accumulator once per group (16 FMAs) instead of once per weight.  Warps of a CTA are reduced through shared
// memory in a fixed order; CTAs along k (S <= 8) form a thread-block cluster and add up their tiles through
// distributed shared memory, for S > 8 they write fp32 partials to scratch and the last one to arrive (atomic ticket,
// no spinning) adds them in a fixed order -> deterministic results, no inter-CTA waits outside a cluster barrier.
// Every launch is a programmatic dependent: it starts its weight stream, releases its own dependents and only then
// waits for the producer of its activations.
//
// Grouped launches.  Up to four projections that read the same activations form one launch: their 64-column blocks
// are laid side by side in one virtual column space (block by block for q/k/v; gate and up blocks interleaved for a
// SwiGLU pair, so that a CTA holds a gate block and its up partner and the epilogue can form silu(gate) * up).
// The epilogue also adds the bias and an optional residual.
//
// Tensor parallelism.  The same epilogue carries the cross-GPU steps of a sharded layer (CommView): the sum of a
// row-parallel shard over the ranks and the gather of a column-parallel shard into every rank's feature area, both as
// epoch-tagged 8-byte words stored into the consumer's memory, every wait bounded.
//
// Roofline: HBM.  Algorithmic bytes per launch = sum over projections of k*n/2 + (k/128)*n*2 + m*n_out*2, + m*k*2.
#include "common.cuh"
#include "linear_internal.cuh"
#include "tma.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

namespace uniql {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;
constexpr int kRedStride = 68;  // floats per row of a warp's 64-column reduction tile (+4: conflict-free scatter)

#ifndef UNIQL_GEMV_CTAS_MT1
#define UNIQL_GEMV_CTAS_MT1 2
#endif
constexpr int kCtasMt1 = UNIQL_GEMV_CTAS_MT1;   // resident CTAs per SM for the m <= 8 variant
constexpr int kXsPad = 16;         // halves of padding per staged activation row (keeps LDS.64 conflict-free)

struct GemvProj {
  const uint4* S;       // permuted scales, row g has N/8 uint4
  const __half* bias;
  __half* D;
  int64_t ldd;
  int N, n_out;
};

struct GemvParams {
  CUtensorMap wmap[kMaxProj];
  GemvProj proj[kMaxProj];
  int vb_start[kMaxProj + 1];   // first virtual block of each projection (plain order)
  const __half* A;
  int64_t lda;
  const __half* residual;       // fp16 [M, n_out] added to the rounded result, or nullptr
  int64_t ldr;
  int M, Nv, KT, nblk, nproj, swiglu;   // Nv = 64 * nblk: width of the virtual column space
  int WN, WK, log_wn, S_split, GCH, R;
  int xs_stride;        // halves per staged activation row (GCH*128 + kXsPad)
  int xs_rows;          // staged rows per warp row: min(M, 8*MT) + 1 (the extra row stays zero)
  int stage_corr;       // 1: the offset term of every staged group is summed while staging (M <= 4: cheaper than the
                        // extra MMA per packed row); 0: it comes from that MMA (the sums grow with the row count)
  float* partials;      // [S_split][M][Nv]
  int* counters;        // [gridDim.x], zero on entry, zero on exit
  int* status_word;
  int cluster;          // 1: the S_split CTAs of a column group form a thread-block cluster and reduce through DSMEM
  int ctile_off;        // byte offset of this CTA's reduced tile in shared memory (cluster mode)
  const unsigned char* pf_ptr[4];   // byte ranges to pull into L2 when this launch's weight stream ends
  long long pf_lines[4];
  int npf;
  CommView cv;          // tensor parallelism: cross-GPU sum of a row-parallel shard / feature gather of a column shard
};

constexpr int kGemvSpinLimit = 1 << 22;   // polls of a word another GPU has to write before giving up

__device__ __forceinline__ void gemv_st_word(uint2* p, uint32_t data, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 gemv_ld_word2(const uint2* p) {   // two adjacent {data, epoch} words
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// virtual block -> (projection, block inside it)
__device__ __forceinline__ void gemv_proj_of(const GemvParams& p, int vb, int& pi, int& lb) {
  if (p.swiglu) {
    pi = vb & 1;
    lb = vb >> 1;
    return;
  }
  pi = 0;
#pragma unroll
  for (int i = 1; i < kMaxProj; ++i)
    if (i < p.nproj && vb >= p.vb_start[i]) pi = i;
  lb = vb - p.vb_start[pi];
}

// One quantisation group (8 packed rows) of one 64-column block, read from this warp's ring slot.
// Nibbles are turned into fp16 values (1024 + q) and (64 + q) by a single LOP3 each; the offsets are taken out again
// by starting the group's accumulators at  -sum_k (off_k + 8) x_k  (off_k = 1024 for k % 16 < 8, else 64):
//   sum_k (off_k + q) x  -  sum_k (off_k + 8) x  =  sum_k (q - 8) x.
// That starting value depends only on the activations; it is computed once per group when they are staged (ncorr).
// Activations are staged so that a lane's (b0, b1) fragment of packed row u is 8 contiguous bytes at xptr + 32u.
template <int MT>
__device__ __forceinline__ void gemv_group_full(const uint8_t* slot_ptr, float (&accg)[MT][4][4], const uint8_t* xptr,
                                                uint32_t x_tile_stride, const float* ncorr_lane) {
  float2 nc[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) nc[t] = *reinterpret_cast<const float2*>(ncorr_lane + 8 * t);
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint4 w4 = *reinterpret_cast<const uint4*>(slot_ptr + u * 512);
    uint2 b[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) b[t] = *reinterpret_cast<const uint2*>(xptr + t * x_tile_stride + u * 32);
    const uint32_t wq[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t a[4];
      const uint32_t q = wq[j], qs = wq[j] >> 8;
      a[0] = lop3_and_or(q, 0x000f000fu, 0x64006400u);     // n = 16j+g,   k = 2c, 2c+1    : 1024 + q
      a[2] = lop3_and_or(q, 0x00f000f0u, 0x54005400u);     // n = 16j+g,   k = 2c+8, 2c+9  :   64 + q
      a[1] = lop3_and_or(qs, 0x000f000fu, 0x64006400u);    // n = 16j+g+8, k = 2c, 2c+1
      a[3] = lop3_and_or(qs, 0x00f000f0u, 0x54005400u);    // n = 16j+g+8, k = 2c+8, 2c+9
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (u == 0) mma_m16n8k16_init(accg[t][j], a, b[t].x, b[t].y, nc[t].x, nc[t].y);
        else mma_m16n8k16(accg[t][j], a, b[t].x, b[t].y);
      }
    }
  }
}

// Same for a group that is only partly inside the warp's k-range [w0, w1): rows are predicated and the offset term
// is accumulated for the rows actually used, with an MMA whose 16-row operand is the constant (1032 | 72).
template <int MT>
__device__ __forceinline__ void gemv_group_partial(const uint8_t* slot_ptr, float (&accg)[MT][4][4], const uint8_t* xptr,
                                                   uint32_t x_tile_stride, int kt_base, int w0, int w1) {
  const uint32_t kcorr[4] = {0x64086408u, 0x64086408u, 0x54805480u, 0x54805480u};   // 1032, 1032, 72, 72
  float corr[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int r = 0; r < 4; ++r) corr[t][r] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) accg[t][j][r] = 0.f;
  }
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    if (kt_base + u >= w0 && kt_base + u < w1) {
      const uint4 w4 = *reinterpret_cast<const uint4*>(slot_ptr + u * 512);
      uint2 b[MT];
#pragma unroll
      for (int t = 0; t < MT; ++t) b[t] = *reinterpret_cast<const uint2*>(xptr + t * x_tile_stride + u * 32);
#pragma unroll
      for (int t = 0; t < MT; ++t) mma_m16n8k16(corr[t], kcorr, b[t].x, b[t].y);
      const uint32_t wq[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a[4];
        const uint32_t q = wq[j], qs = wq[j] >> 8;
        a[0] = lop3_and_or(q, 0x000f000fu, 0x64006400u);
        a[2] = lop3_and_or(q, 0x00f000f0u, 0x54005400u);
        a[1] = lop3_and_or(qs, 0x000f000fu, 0x64006400u);
        a[3] = lop3_and_or(qs, 0x00f000f0u, 0x54005400u);
#pragma unroll
        for (int t = 0; t < MT; ++t) mma_m16n8k16(accg[t][j], a, b[t].x, b[t].y);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) accg[t][j][r] -= corr[t][r];
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes from the shared memory of CTA `rank` of this cluster (distributed shared memory)
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

template <int MT>
__global__ void __launch_bounds__(kGemvThreads, MT == 1 ? kCtasMt1 : 2)
w4a16_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ int s_is_last;
  __shared__ uint32_t s_repoch[kGemvWarps], s_gepoch[kGemvWarps];   // per block of the CTA: epoch of this call's words
  __shared__ __align__(8) uint64_t s_bars[kGemvWarps * 4];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int wn = warp & (p.WN - 1), wk = warp >> p.log_wn;
  const int blk = blockIdx.x * p.WN + wn;          // block in the launch's virtual column space
  const bool active = blk < p.nblk;
  int pi = 0, lb = 0;                              // its projection and its block inside that projection
  if (active) gemv_proj_of(p, blk, pi, lb);
  const CUtensorMap* wmap = &p.wmap[pi];

  // k-range of this CTA, then of this warp row (contiguous, balanced to one packed row).
  const unsigned ukt = (unsigned)p.KT, us = (unsigned)p.S_split, uwk = (unsigned)p.WK;   // KT * S_split < 2^31
  const int cta_k0 = (int)(ukt * blockIdx.y / us);
  const int cta_k1 = (int)(ukt * (blockIdx.y + 1) / us);
  const int rw0 = cta_k0 + (int)((unsigned)(cta_k1 - cta_k0) * (unsigned)wk / uwk);
  const int rw1 = cta_k0 + (int)((unsigned)(cta_k1 - cta_k0) * (unsigned)(wk + 1) / uwk);
  const int g0 = rw0 >> 3, g1 = (rw1 + 7) >> 3;   // quantisation groups touched (8 packed rows each)
  const int w0 = active ? rw0 : 0, w1 = active ? rw1 : 0;   // empty range for warps past the last block
  const bool has_work = w0 < w1;

  // ---- shared memory carve-up: [rings: 8 warps x R slots x 4 KB][staged activations] ----
  const uint32_t ring_base = smem_addr(smem_raw) + warp * p.R * kSlotBytes;
  const uint32_t bar0 = smem_addr(&s_bars[warp * 4]);
  __half* xs_all = reinterpret_cast<__half*>(smem_raw + (size_t)kGemvWarps * p.R * kSlotBytes);
  __half* xs = xs_all + (size_t)wk * p.xs_rows * p.xs_stride;
  // per warp row: -(offset term) of every staged group and batch row, [GCH][16] floats (rows >= M stay zero)
  float* ncorr = reinterpret_cast<float*>(xs_all + (size_t)p.WK * p.xs_rows * p.xs_stride) + (size_t)wk * p.GCH * 16;

  const uint64_t pol = make_evict_first_policy();
  const uint32_t srow_u4 = (uint32_t)(p.proj[pi].N >> 3);
  const uint4* sptr = p.proj[pi].S + (size_t)lb * 8 + g + (size_t)g0 * srow_u4;

  if (lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(wmap) : "memory");   // hide the descriptor fetch of the first tile
    for (int s = 0; s < p.R; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  // ---- start streaming weights before anything else: one TMA tile per group and 64-column block ----
  if (has_work && lane == 0) {
    for (int s = 0; s < p.R; ++s)
      if (g0 + s < g1) {
        mbar_expect_tx(bar0 + s * 8, kSlotBytes);
        tma_load_slot(ring_base + s * kSlotBytes, wmap, lb * 128, 8 * (g0 + s), bar0 + s * 8, pol);
      }
  }
  // Let the next kernel in the stream start its own weight prefetch, then wait for the producer of A.
  pdl_launch_dependents();
  pdl_wait();
  if ((p.cv.reduce || p.cv.gather_out) && tid < p.WN) {
    // epoch counters live on the device (CUDA-graph replay safe), one per 64-column block (per gate/up pair)
    const int vb = blockIdx.x * p.WN + tid;
    if (vb < p.nblk) {
      const size_t unit = (size_t)(p.swiglu ? vb >> 1 : vb);
      if (p.cv.reduce)
        s_repoch[tid] = *reinterpret_cast<const volatile uint32_t*>(p.cv.bufs[p.cv.rank] + p.cv.reduce_epoch_off + 4 * unit) + 1;
      // feature gather: one epoch per launch (this rank's gather counter + 1); the counter itself is advanced by the
      // consumer of the gathered row (hadamard_split_feat_kernel), which runs between two producer launches
      if (p.cv.gather_out)
        s_gepoch[tid] = *reinterpret_cast<const volatile uint32_t*>(p.cv.bufs[p.cv.rank] + p.cv.gather_epoch_off) + 1;
    }
  }

  const int row_threads = p.WN * 32;
  const int row_tid = wn * 32 + lane;
  const int m_staged = p.xs_rows - 1;                 // real rows staged by this kernel (M, at most 8*MT)
  // the extra row is read by MMA lanes whose batch row does not exist: clear it once
  for (int v = row_tid; v < p.xs_stride / 8; v += row_threads)
    *reinterpret_cast<uint4*>(xs + (size_t)m_staged * p.xs_stride + v * 8) = make_uint4(0, 0, 0, 0);
  for (int v = row_tid; v < p.GCH * 16; v += row_threads) ncorr[v] = 0.f;
  // this lane's B-fragment origin for batch tile 0 and the distance to tile 1 (bytes)
  const int row_t0 = min(g, m_staged), row_t1 = min(8 + g, m_staged);
  const uint8_t* xl = reinterpret_cast<const uint8_t*>(xs) + (size_t)row_t0 * p.xs_stride * 2 + c * 8;
  const uint32_t x_tile_stride = (uint32_t)(row_t1 - row_t0) * p.xs_stride * 2;

  float acc[MT][4][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[t][j][r] = 0.f;

  int chunk_pos = 0;   // group index inside the staged chunk
  int slot = 0;
  uint32_t parity = 0;
  bool timed_out = false;
  for (int gi = g0; gi < g1; ++gi) {
    // ---- stage the next chunk of activations for this warp row (GCH groups = GCH*128 k-values) ----
    // Layout per row: packed row u occupies 32 bytes holding, for c = 0..3, the halves (2c, 2c+1, 2c+8, 2c+9).
    if (chunk_pos == 0) {
      asm volatile("bar.sync %0, %1;" ::"r"(wk + 1), "r"(row_threads));
      const int blocks_per_row = (min(gi + p.GCH, g1) - gi) * 8;   // 16-value blocks per row
      const __half* src = p.A + (size_t)gi * 128;
      if (!(MT == 1 && p.stage_corr)) {
        // no offset sums to form: the (row, block) pairs are dealt out flat over the lanes, FL loads in flight each
        constexpr int FL = MT == 1 ? 4 : 2;
        const int nitems = blocks_per_row * m_staged;
        for (int i0 = 0; i0 < nitems; i0 += FL * row_threads) {
          uint4 lo[FL], hi[FL];
          int dst[FL];
#pragma unroll
          for (int i = 0; i < FL; ++i) {
            const int item = i0 + i * row_threads + row_tid;
            dst[i] = -1;
            if (item < nitems) {
              const int r = item / blocks_per_row, v = item - r * blocks_per_row;
              const __half* s16 = src + (size_t)r * p.lda + v * 16;
              lo[i] = ld_nc16(s16);
              hi[i] = ld_nc16(s16 + 8);
              dst[i] = r * p.xs_stride + v * 16;
            }
          }
#pragma unroll
          for (int i = 0; i < FL; ++i)
            if (dst[i] >= 0) {
              uint4* d = reinterpret_cast<uint4*>(xs + dst[i]);
              d[0] = make_uint4(lo[i].x, hi[i].x, lo[i].y, hi[i].y);
              d[1] = make_uint4(lo[i].z, hi[i].z, lo[i].w, hi[i].w);
            }
        }
      } else
      // every lane takes part in the shuffles below: warp-uniform trip count, out-of-range blocks contribute zero
      // (rows are loaded two at a time into registers; staging all rows at once through asynchronous copies was
      // measured and changed nothing at 8 rows while costing 1 % at one row)
      for (int v0 = 0; v0 < blocks_per_row; v0 += row_threads) {
        const int v = v0 + row_tid;
        const bool vin = v < blocks_per_row;
        constexpr int RB = MT == 1 ? 2 : 4;   // rows loaded together (independent requests in flight)
        for (int r0 = 0; r0 < m_staged; r0 += RB) {
          uint4 lo[RB], hi[RB];
#pragma unroll
          for (int i = 0; i < RB; ++i) {
            lo[i] = make_uint4(0, 0, 0, 0);
            hi[i] = make_uint4(0, 0, 0, 0);
            if (vin && r0 + i < m_staged) {
              const __half* s16 = src + (size_t)(r0 + i) * p.lda + v * 16;
              lo[i] = ld_nc16(s16);
              hi[i] = ld_nc16(s16 + 8);
            }
          }
#pragma unroll
          for (int i = 0; i < RB; ++i) {
            if (vin && r0 + i < m_staged) {
              uint4* d = reinterpret_cast<uint4*>(xs + (size_t)(r0 + i) * p.xs_stride + v * 16);
              d[0] = make_uint4(lo[i].x, hi[i].x, lo[i].y, hi[i].y);
              d[1] = make_uint4(lo[i].z, hi[i].z, lo[i].w, hi[i].w);
            }
            if (MT != 1) continue;   // (not reached with two batch tiles: see the branch above)
            // offset term of this 16-value block: 1032 * (sum of k % 16 < 8) + 72 * (sum of k % 16 >= 8)
            const __half2* hl = reinterpret_cast<const __half2*>(&lo[i]);
            const __half2* hh = reinterpret_cast<const __half2*>(&hi[i]);
            float sl = 0.f, sh = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 fl = __half22float2(hl[e]), fh = __half22float2(hh[e]);
              sl += fl.x + fl.y;
              sh += fh.x + fh.y;
            }
            float part = 1032.f * sl + 72.f * sh;
            // the 8 blocks of a group sit in 8 consecutive lanes: fixed-order butterfly sum
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            if (vin && (lane & 7) == 0 && r0 + i < m_staged) ncorr[(v >> 3) * 16 + r0 + i] = -part;
          }
        }
      }
      asm volatile("bar.sync %0, %1;" ::"r"(wk + 1), "r"(row_threads));
    }
    if (has_work) {
      // this group's 8 scales; the load is covered by the group's MMAs
      const uint4 s_cur = ld_nc16(sptr + (size_t)(gi - g0) * srow_u4);

      float accg[MT][4][4];
      if (!mbar_wait(bar0 + slot * 8, parity)) timed_out = true;
      const uint8_t* slot_addr = smem_raw + (size_t)(warp * p.R + slot) * kSlotBytes + lane * 16;
      const uint8_t* xg = xl + chunk_pos * 256;
      // m <= 8: the offset term was computed while staging; m > 8: staging 16 rows is already the longer part of
      // the prologue, so the offset term rides on the tensor pipe there
      if (MT == 1 && p.stage_corr && 8 * gi >= w0 && 8 * gi + 8 <= w1)
        gemv_group_full<MT>(slot_addr, accg, xg, x_tile_stride, ncorr + chunk_pos * 16 + 2 * c);
      else
        gemv_group_partial<MT>(slot_addr, accg, xg, x_tile_stride, 8 * gi, w0, w1);
      // the slot has been read by every lane: hand it back to the copy engine
      __syncwarp();
      if (lane == 0 && gi + p.R < g1) {
        mbar_expect_tx(bar0 + slot * 8, kSlotBytes);
        tma_load_slot(ring_base + slot * kSlotBytes, wmap, lb * 128, 8 * (gi + p.R), bar0 + slot * 8, pol);
      }

      // ---- apply this group's scales: lane holds s[64blk + 8g + 2j + b] for j=0..3, b=0..1 ----
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
    if (++chunk_pos == p.GCH) chunk_pos = 0;
    if (++slot == p.R) { slot = 0; parity ^= 1; }
  }
  if (timed_out && lane == 0 && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);

  // This CTA's weight stream has ended: ask L2 for its share of the weights the following launches will stream, so
  // that HBM keeps working while this launch reduces and drains (plain per-line prefetch hints).
  for (int r = 0; r < p.npf; ++r) {
    const long long nthreads_all = (long long)gridDim.x * gridDim.y * kGemvThreads;
    const long long gtid = ((long long)blockIdx.y * gridDim.x + blockIdx.x) * kGemvThreads + tid;
    for (long long l = gtid; l < p.pf_lines[r]; l += nthreads_all)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.pf_ptr[r] + l * 128));
  }

  // ---- reduce the WK warp rows through shared memory (fixed order) ----
  __syncthreads();   // every copy issued has been consumed; rings and staged activations can be reused
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

  // An output item is 4 adjacent columns of one batch row.  Plain launches: every column of the CTA.  SwiGLU pair:
  // the CTA's blocks alternate gate, up, gate, up ...: an item is 4 columns of a gate block, and its partner sits one
  // block (64 columns) to the right.
  const int sw = p.swiglu;
  const int log_cols4 = p.log_wn + 4 - sw;            // log2(output columns of the CTA / 4)
  const int n_base = blockIdx.x * (p.WN * 64);        // first virtual column of the CTA
  const int items = p.M << log_cols4;
  const bool direct = (p.S_split == 1);
  auto item_col = [&](int idx, int& m, int& col) {    // CTA-local column (of the gate block for a pair)
    m = idx >> log_cols4;
    const int oc = (idx & ((1 << log_cols4) - 1)) * 4;
    col = sw ? ((oc >> 6) << 7) + (oc & 63) : oc;
  };
  auto warp_sum = [&](int m, int col) {               // the CTA's WK warp rows of (m, col..col+3), in order
    const int wn_i = col >> 6, nl = col & 63;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < p.WK; ++k) {
      const float4 t4 = *reinterpret_cast<const float4*>(red + ((size_t)((k << p.log_wn) + wn_i) * (8 * MT) + m) * kRedStride + nl);
      v.x += t4.x; v.y += t4.y; v.z += t4.z; v.w += t4.w;
    }
    return v;
  };
  // bias, SwiGLU product, residual, fp16 store of 4 columns starting at virtual column nv
  auto store_out = [&](int m, int nv, float4 v, float4 v2) {
    const int vb = nv >> 6;
    if (vb >= p.nblk) return;
    int qi, qb;
    gemv_proj_of(p, vb, qi, qb);
    const GemvProj& pr = p.proj[qi];
    const int n = qb * 64 + (nv & 63);
    if (n >= pr.n_out) return;
    float a[4] = {v.x, v.y, v.z, v.w};
    float u[4] = {v2.x, v2.y, v2.z, v2.w};
    __half h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (n + e >= pr.n_out) { h[e] = __float2half_rn(0.f); continue; }
      if (pr.bias) a[e] += __half2float(pr.bias[n + e]);
      h[e] = __float2half_rn(a[e]);
      if (sw) {
        // act_fn(gate) * up with the roundings of the separate modules: fp16 gate, fp16 up, fp16 SiLU, fp16 product
        if (p.proj[1].bias) u[e] += __half2float(p.proj[1].bias[n + e]);
        const __half uh = __float2half_rn(u[e]);
        const float gf = __half2float(h[e]);
        const __half ah = __float2half_rn(gf / (1.0f + expf(-gf)));
        h[e] = __float2half_rn(__half2float(ah) * __half2float(uh));
      }
      if (p.residual) h[e] = __float2half_rn(__half2float(h[e]) + __half2float(p.residual[(size_t)m * p.ldr + n + e]));
    }
    if (p.cv.gather_out) {
      // column shard of a tensor-parallel layer: the finished columns also go, as epoch-tagged words, into every rank's
      // feature area (only real columns travel; n_out is even)
      const uint32_t ep = s_gepoch[(nv - n_base) >> 6];
      const size_t word = ((size_t)(ep & 1u) * 16 + m) * (size_t)(p.cv.feat_cap >> 1) + (size_t)((p.cv.col_offset + n) >> 1);
      const uint32_t w0 = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
      const uint32_t w1 = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
      for (int r = 0; r < p.cv.world; ++r) {
        uint2* dst = reinterpret_cast<uint2*>(p.cv.bufs[r] + p.cv.gather_off) + word;
        if (n + 1 < pr.n_out) gemv_st_word(dst, w0, ep);
        if (n + 3 < pr.n_out) gemv_st_word(dst + 1, w1, ep);
      }
    }
    __half* d = pr.D + (size_t)m * pr.ldd + n;
    if (n + 3 < pr.n_out && ((reinterpret_cast<uintptr_t>(d) & 7u) == 0)) {
      uint2 pk;
      pk.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
      pk.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
      *reinterpret_cast<uint2*>(d) = pk;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (n + e < pr.n_out) d[e] = h[e];
    }
  };

  // Row-parallel shard of a tensor-parallel layer: where a rank would store its fp16 result it stores the partial, as
  // epoch-tagged words, into every rank's staging block (addressed per 64-column block: 16 rows x 32 words) ...
  bool wait_failed = false;
  auto push4 = [&](int m, int nv, float4 v) {
    const int vb = nv >> 6;
    if (vb >= p.nblk) return;
    const uint32_t ep = s_repoch[(nv - n_base) >> 6];
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    const size_t word = (size_t)vb * kFuseBlockWords + (size_t)m * 32 + ((nv & 63) >> 1);
    const size_t slot = ((size_t)(ep & 1u) * p.cv.world + p.cv.rank) * (size_t)p.cv.block_cap * kFuseBlockWords + word;
    for (int r = 0; r < p.cv.world; ++r) {
      uint2* dst = reinterpret_cast<uint2*>(p.cv.bufs[r] + p.cv.reduce_off) + slot;
      gemv_st_word(dst, *reinterpret_cast<const uint32_t*>(&lo), ep);
      gemv_st_word(dst + 1, *reinterpret_cast<const uint32_t*>(&hi), ep);
    }
  };
  // ... and then adds up the words of all ranks that arrived in its own block (bounded wait, rank order, fp32: the same
  // bits on every rank)
  auto gather4 = [&](int m, int nv) {
    float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const int vb = nv >> 6;
    if (vb >= p.nblk) return acc4;
    const uint32_t ep = s_repoch[(nv - n_base) >> 6];
    const size_t word = (size_t)vb * kFuseBlockWords + (size_t)m * 32 + ((nv & 63) >> 1);
    const uint2* base = reinterpret_cast<const uint2*>(p.cv.bufs[p.cv.rank] + p.cv.reduce_off) +
                        (size_t)(ep & 1u) * p.cv.world * (size_t)p.cv.block_cap * kFuseBlockWords + word;
    // the first look at every rank's words goes out together (one round trip instead of one per rank); a word that
    // has not arrived yet is then polled on its own
    const size_t rstride = (size_t)p.cv.block_cap * kFuseBlockWords;
    uint4 w[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.cv.world) w[r] = gemv_ld_word2(base + (size_t)r * rstride);
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.cv.world) {
        int spin = 0;
        while ((w[r].y != ep || w[r].w != ep) && !wait_failed) {
          if (++spin > kGemvSpinLimit) { wait_failed = true; break; }
          w[r] = gemv_ld_word2(base + (size_t)r * rstride);
        }
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[r].x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w[r].z));
        acc4.x += a.x; acc4.y += a.y; acc4.z += b.x; acc4.w += b.y;
      }
    return acc4;
  };
  // finishes output items [i0, i1) whose values `sumfn(m, col)` delivers
  auto finish_items = [&](int i0, int i1, auto&& sumfn) {
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!p.cv.reduce) {
      for (int idx = i0 + tid; idx < i1; idx += kGemvThreads) {
        int m, col;
        item_col(idx, m, col);
        if (n_base + col >= p.Nv) continue;
        store_out(m, n_base + col, sumfn(m, col), sw ? sumfn(m, col + 64) : zero4);
      }
      return;
    }
    for (int idx = i0 + tid; idx < i1; idx += kGemvThreads) {
      int m, col;
      item_col(idx, m, col);
      if (n_base + col >= p.Nv) continue;
      push4(m, n_base + col, sumfn(m, col));
    }
    for (int idx = i0 + tid; idx < i1; idx += kGemvThreads) {
      int m, col;
      item_col(idx, m, col);
      if (n_base + col >= p.Nv) continue;
      store_out(m, n_base + col, gather4(m, n_base + col), zero4);
    }
    if (wait_failed && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);
  };
  // once every item of the CTA's blocks is finished, their epoch counters advance (one thread per block)
  auto advance_epochs = [&]() {
    if (p.cv.reduce && tid < p.WN) {
      const int vb = blockIdx.x * p.WN + tid;
      if (vb < p.nblk) {
        const size_t unit = (size_t)(p.swiglu ? vb >> 1 : vb);
        *reinterpret_cast<volatile uint32_t*>(p.cv.bufs[p.cv.rank] + p.cv.reduce_epoch_off + 4 * unit) = s_repoch[tid];
      }
    }
  };

  // ---- split-k inside a thread-block cluster: partial tiles stay in shared memory, every CTA of the cluster adds
  // up one slice of the tile by reading its peers' shared memory in rank order (no global scratch, no ticket) ----
  if (p.cluster && !direct) {
    float* ctile = reinterpret_cast<float*>(smem_raw + p.ctile_off);
    const int cta_cols = p.WN * 64;
    const int all_items = p.M << (p.log_wn + 4);
    for (int idx = tid; idx < all_items; idx += kGemvThreads) {
      const int m = idx >> (p.log_wn + 4), col = (idx & ((1 << (p.log_wn + 4)) - 1)) * 4;
      *reinterpret_cast<float4*>(ctile + (size_t)m * cta_cols + col) = warp_sum(m, col);
    }
    cluster_sync_all();
    const int rank = blockIdx.y;                  // cluster = the S_split CTAs with the same blockIdx.x
    const int i0 = (int)((int64_t)items * rank / p.S_split), i1 = (int)((int64_t)items * (rank + 1) / p.S_split);
    const uint32_t ctile_addr = smem_addr(ctile);
    auto cluster_sum = [&](int m, int col) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const uint32_t off = ctile_addr + (uint32_t)((m * cta_cols + col) * 4);
      // all peers' tiles are requested before the first is added (2 <= S_split <= 8): one remote round trip, not S
      float4 t4[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.S_split) t4[r] = ld_dsmem_f4(off, (uint32_t)r);
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.S_split) { v.x += t4[r].x; v.y += t4[r].y; v.z += t4[r].z; v.w += t4[r].w; }
      return v;
    };
    finish_items(i0, i1, cluster_sum);
    cluster_sync_all();                           // peers may still be reading this CTA's tile
    if (rank == 0) advance_epochs();
    return;
  }

  if (direct) {
    finish_items(0, items, warp_sum);
    __syncthreads();
    advance_epochs();
    return;
  }

  // ---- split-k through scratch: every CTA writes its partial sums, the last CTA of the column group to finish
  // (atomic ticket, no spinning) adds them in a fixed order ----
  {
    const int all_items = p.M << (p.log_wn + 4);
    for (int idx = tid; idx < all_items; idx += kGemvThreads) {
      const int m = idx >> (p.log_wn + 4), col = (idx & ((1 << (p.log_wn + 4)) - 1)) * 4;
      const int nv = n_base + col;
      if (nv >= p.Nv) continue;
      *reinterpret_cast<float4*>(p.partials + ((size_t)blockIdx.y * p.M + m) * p.Nv + nv) = warp_sum(m, col);
    }
  }
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
  const size_t slab4 = ((size_t)p.M * p.Nv) >> 2;
  auto partial_sum = [&](int m, int nv) {
    const float4* src = reinterpret_cast<const float4*>(p.partials + (size_t)m * p.Nv + nv);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < p.S_split; s += 8) {      // up to 8 independent L2 loads in flight, summed in order
      float4 t4[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        t4[i] = (s + i < p.S_split) ? __ldcg(src + (size_t)(s + i) * slab4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { v.x += t4[i].x; v.y += t4[i].y; v.z += t4[i].z; v.w += t4[i].w; }
    }
    return v;
  };
  finish_items(0, items, [&](int m, int col) { return partial_sum(m, n_base + col); });
  __syncthreads();
  advance_epochs();
}

// ------------------------------------------------------------------ host side
static int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

struct GemvPlan {
  int WN, WK, S, GCH, MT, R, xs_rows;
  int cluster, ctile_off;
  size_t smem;
  size_t partial_bytes;
};

// n: width of the launch's virtual column space (all projections side by side).  pair: the blocks alternate gate / up,
// so a CTA must hold an even number of them.
// The tuning overrides are read from the environment once per process (a getenv per launch is a scan of the whole
// environment block).
struct GemvEnv {
  int slots, wn, s, r, cluster, stage_corr_rows;
};
static const GemvEnv& gemv_env() {
  static const GemvEnv e = {env_int("UNIQL_B200_GEMV_SLOTS", 0), env_int("UNIQL_B200_GEMV_WN", 0),
                            env_int("UNIQL_B200_GEMV_S", 0), env_int("UNIQL_B200_GEMV_R", 0),
                            env_int("UNIQL_B200_CLUSTER", 1), env_int("UNIQL_B200_GEMV_STAGE_CORR_ROWS", 4)};
  return e;
}

static GemvPlan make_gemv_plan(int64_t m, int64_t n, int64_t k, bool pair);

// Plans are a pure function of (m, n, k, pair): the last few are remembered so that an eager decode loop does not run
// the cost model on every launch.
static GemvPlan plan_gemv(int64_t m, int64_t n, int64_t k, bool pair) {
  struct Entry { int64_t m, n, k; bool pair; GemvPlan plan; };
  static std::mutex mu;
  static std::vector<Entry> cache;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (const Entry& e : cache)
      if (e.m == m && e.n == n && e.k == k && e.pair == pair) return e.plan;
  }
  const GemvPlan plan = make_gemv_plan(m, n, k, pair);
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() >= 256) cache.clear();
  cache.push_back({m, n, k, pair, plan});
  return plan;
}

static GemvPlan make_gemv_plan(int64_t m, int64_t n, int64_t k, bool pair) {
  GemvPlan best{};
  const int MT = m <= 8 ? 1 : 2;
  const int nblk = (int)(n / 64), KT = (int)(k / 16), NG = KT / 8;
  const int ctas_per_sm = MT == 1 ? kCtasMt1 : 2;
  const int slots = device_info().sm_count * (gemv_env().slots > 0 ? gemv_env().slots : ctas_per_sm);
  double best_cost = 1e30;
  for (int WN = 8; WN >= (pair ? 2 : 1); WN >>= 1) {
    const int WK = kGemvWarps / WN;
    const int groups = (nblk + WN - 1) / WN;
    const double waste = (double)(groups * WN) / nblk;   // idle warps in the last column group
    const int smax = KT / WK < 1 ? 1 : (KT / WK > 64 ? 64 : KT / WK);
    for (int S = 1; S <= smax; ++S) {
      const int64_t ctas = (int64_t)groups * S;
      const int64_t waves = (ctas + slots - 1) / slots;
      const int splits = S * WK;
      // packed rows streamed by the busiest warp; a k-range that is not a whole number of quantisation
      // groups pays for the partly used first/last group through the slower predicated path
      const int len = (KT + splits - 1) / splits;
      const bool aligned = (NG % splits) == 0;
      const double eff_len = aligned ? len : len + 14.0;
      // cost in "packed rows per warp": streamed rows + fixed latency per wave + split-k reduction
      double cost = (double)waves * (eff_len + 12.0) * waste + (S > 1 ? 6.0 + 0.35 * S : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best.WN = WN; best.WK = WK; best.S = S;
      }
    }
  }
  const int ov_wn = gemv_env().wn, ov_s = gemv_env().s;
  if ((ov_wn == 1 && !pair) || ov_wn == 2 || ov_wn == 4 || ov_wn == 8) { best.WN = ov_wn; best.WK = kGemvWarps / ov_wn; }
  if (ov_s >= 1) best.S = ov_s;
  if (best.S > KT) best.S = KT;
  // Shared memory per CTA: rings = 8 warps x R slots x 4 KB, then the staged activations
  // = WK warp rows x (rows + 1) x (GCH*128 + pad) halves.  Budget: 3 CTAs per SM for m <= 8, else 2.
  const int rows = (int)(m < 8 * MT ? m : 8 * MT) + 1;
  const size_t budget = (MT == 1 && kCtasMt1 == 3 ? 74 : 110) * 1024;
  const size_t xs_min = (size_t)best.WK * rows * (128 + kXsPad) * 2 + (size_t)best.WK * 8 * 64;
  int R = (int)((budget - xs_min) / (kGemvWarps * kSlotBytes));
  // two slots per warp measured faster than three for m <= 8 (39.1 vs 41.6 us per Llama-3.1-8B layer)
  const int r_max = MT == 1 ? 2 : 3;
  if (R > r_max) R = r_max;
  if (R < 1) R = 1;
  const int ov_r = gemv_env().r;
  if (ov_r >= 1 && ov_r <= 4) R = ov_r;
  const size_t ring_bytes = (size_t)kGemvWarps * R * kSlotBytes;
  const size_t left = budget > ring_bytes ? budget - ring_bytes : 0;
  // per group and warp row: rows * 128 halves of activations + 16 floats of offset terms
  int gch = (int)((left > (size_t)best.WK * rows * 2 * kXsPad ? left - (size_t)best.WK * rows * 2 * kXsPad : 0) /
                  ((size_t)best.WK * (rows * 256 + 64)));
  if (gch < 1) gch = 1;
  if (gch > 8) gch = 8;
  best.GCH = gch;
  best.MT = MT;
  best.R = R;
  best.xs_rows = rows;
  const size_t xs_bytes = (size_t)best.WK * rows * (gch * 128 + kXsPad) * 2 + (size_t)best.WK * gch * 64;
  const size_t red_bytes = (size_t)kGemvWarps * 8 * MT * kRedStride * 4;
  best.smem = ring_bytes + xs_bytes > red_bytes ? ring_bytes + xs_bytes : red_bytes;
  // cluster mode (2 <= S <= 8): the CTA's reduced tile lives behind the warp reduction buffer
  best.cluster = (gemv_env().cluster && best.S >= 2 && best.S <= 8) ? 1 : 0;
  best.ctile_off = (int)((red_bytes + 1023) / 1024 * 1024);
  if (best.cluster) {
    const size_t need = (size_t)best.ctile_off + (size_t)(m < 16 ? m : 16) * best.WN * 64 * 4;
    if (best.smem < need) best.smem = need;
  }
  best.partial_bytes = (best.S > 1 && !best.cluster) ? (size_t)best.S * (size_t)(m < 16 ? m : 16) * n * 4 : 0;
  return best;
}

static int64_t virtual_width(const int64_t* n, int nproj) {
  int64_t w = 0;
  for (int i = 0; i < nproj; ++i) w += n[i];
  return w;
}

// Host-only check of the plan a launch of this shape would get (no device work): the invariants the kernel's index
// arithmetic relies on, and that the k-ranges of its warps tile [0, k/16) exactly once.  0, or the number of the
// failed check; out5 (may be null) receives {WN, S, cluster, dynamic shared memory, partial bytes}.
int gemv_plan_check(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t* out5) {
  if (m < 1 || m > 16 || k <= 0 || k % 128 || nproj < 1 || nproj > kMaxProj) return 1;
  const bool pair = epilogue == UNIQL_EPILOGUE_SWIGLU;
  if (pair && (nproj != 2 || n[0] != n[1])) return 2;
  for (int i = 0; i < nproj; ++i)
    if (n[i] <= 0 || n[i] % 64) return 3;
  const int64_t nv = virtual_width(n, nproj);
  const GemvPlan pl = plan_gemv(m, nv, k, pair);
  if (out5) { out5[0] = pl.WN; out5[1] = pl.S; out5[2] = pl.cluster; out5[3] = (int64_t)pl.smem; out5[4] = (int64_t)pl.partial_bytes; }
  const int KT = (int)(k / 16), nblk = (int)(nv / 64);
  if (!(pl.WN == 1 || pl.WN == 2 || pl.WN == 4 || pl.WN == 8) || pl.WN * pl.WK != kGemvWarps) return 10;
  if (pair && pl.WN < 2) return 11;
  if (pl.S < 1 || pl.S > KT || pl.S > 64) return 12;
  if (pl.cluster && (pl.S < 2 || pl.S > 8)) return 13;
  if (pl.MT != (m <= 8 ? 1 : 2) || pl.R < 1 || pl.R > 4 || pl.GCH < 1 || pl.GCH > 8) return 14;
  if (pl.xs_rows != (int)(m < 8 * pl.MT ? m : 8 * pl.MT) + 1) return 15;
  const int grid_x = (nblk + pl.WN - 1) / pl.WN;
  if ((size_t)grid_x * sizeof(int) > UNIQL_SCRATCH_COUNTER_BYTES) return 16;
  // two CTAs per SM must fit (227 KB of shared memory per SM, 1 KB reserved per CTA, the kernel's static part on top)
  if (pl.smem > 160 * 1024 || 2 * (pl.smem + 2048) > 227 * 1024) return 17;
  const size_t ring_bytes = (size_t)kGemvWarps * pl.R * kSlotBytes;
  const size_t xs_bytes = (size_t)pl.WK * pl.xs_rows * (pl.GCH * 128 + kXsPad) * 2 + (size_t)pl.WK * pl.GCH * 64;
  if (ring_bytes + xs_bytes > pl.smem) return 18;
  if ((size_t)kGemvWarps * 8 * pl.MT * kRedStride * 4 > pl.smem) return 19;
  if (pl.cluster && (size_t)pl.ctile_off + (size_t)m * pl.WN * 64 * 4 > pl.smem) return 20;
  if (pl.partial_bytes != ((pl.S > 1 && !pl.cluster) ? (size_t)pl.S * (size_t)m * nv * 4 : 0)) return 21;
  if (gemv_scratch_bytes(m, k, n, nproj, epilogue) != UNIQL_SCRATCH_COUNTER_BYTES + (pl.partial_bytes + 255) / 256 * 256)
    return 22;
  // the warps' k-ranges, as the kernel computes them: disjoint, in order, covering every packed row once
  int next = 0;
  for (int y = 0; y < pl.S; ++y) {
    const int k0 = (int)((unsigned)KT * (unsigned)y / (unsigned)pl.S), k1 = (int)((unsigned)KT * (unsigned)(y + 1) / (unsigned)pl.S);
    for (int wk = 0; wk < pl.WK; ++wk) {
      const int r0 = k0 + (int)((unsigned)(k1 - k0) * (unsigned)wk / (unsigned)pl.WK);
      const int r1 = k0 + (int)((unsigned)(k1 - k0) * (unsigned)(wk + 1) / (unsigned)pl.WK);
      if (r0 != next || r1 < r0) return 23;
      next = r1;
    }
  }
  if (next != KT) return 24;
  return 0;
}

size_t gemv_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue) {
  if (m < 1 || m > 16 || nproj < 1 || nproj > kMaxProj) return UNIQL_SCRATCH_COUNTER_BYTES;
  const GemvPlan plan = plan_gemv(m, virtual_width(n, nproj), k, epilogue == UNIQL_EPILOGUE_SWIGLU);
  return UNIQL_SCRATCH_COUNTER_BYTES + (plan.partial_bytes + 255) / 256 * 256;
}

// A: the activations the kernel multiplies with (already transformed if the layer has an online Hadamard).
int launch_gemv_group(const DecodeArgs& a, const __half* A, int64_t lda, cudaStream_t stream) {
  if (a.nproj < 1 || a.nproj > kMaxProj || a.m < 1 || a.m > 16 || a.k % 128) return UNIQL_ESHAPE;
  const bool pair = a.epilogue == UNIQL_EPILOGUE_SWIGLU;
  if (pair && (a.nproj != 2 || a.proj[0].n != a.proj[1].n)) return UNIQL_EINVAL;
  int64_t widths[kMaxProj] = {0, 0, 0, 0};
  for (int i = 0; i < a.nproj; ++i) {
    if (a.proj[i].n <= 0 || a.proj[i].n % 64) return UNIQL_ESHAPE;
    widths[i] = a.proj[i].n;
  }
  const int64_t nv = virtual_width(widths, a.nproj);
  const GemvPlan plan = plan_gemv(a.m, nv, a.k, pair);
  GemvParams p;
  memset(&p, 0, sizeof(p));
  int vb = 0;
  for (int i = 0; i < a.nproj; ++i) {
    const DecodeProjArgs& q = a.proj[i];
    int st = cached_weight_map(&p.wmap[i], q.B, q.n, a.k / 16);
    if (st != UNIQL_OK) return st;
    p.proj[i].S = (const uint4*)q.s; p.proj[i].bias = (const __half*)q.bias; p.proj[i].D = (__half*)q.D;
    p.proj[i].ldd = q.ldd; p.proj[i].N = (int)q.n; p.proj[i].n_out = (int)q.n_out;
    p.vb_start[i] = vb;
    vb += (int)(q.n / 64);
  }
  for (int i = a.nproj; i <= kMaxProj; ++i) p.vb_start[i] = vb;
  for (int i = a.nproj; i < kMaxProj; ++i) { p.wmap[i] = p.wmap[0]; p.proj[i] = p.proj[0]; }
  p.A = A; p.lda = lda;
  p.residual = (const __half*)a.residual; p.ldr = a.ldr;
  p.M = (int)a.m; p.Nv = (int)nv; p.KT = (int)(a.k / 16); p.nblk = vb; p.nproj = a.nproj; p.swiglu = pair ? 1 : 0;
  p.WN = plan.WN; p.WK = plan.WK; p.S_split = plan.S; p.GCH = plan.GCH;
  p.log_wn = plan.WN == 1 ? 0 : plan.WN == 2 ? 1 : plan.WN == 4 ? 2 : 3;
  p.xs_stride = plan.GCH * 128 + kXsPad;
  p.R = plan.R; p.xs_rows = plan.xs_rows; p.status_word = a.status_word;
  p.stage_corr = a.m <= gemv_env().stage_corr_rows ? 1 : 0;
  p.cluster = plan.cluster; p.ctile_off = plan.ctile_off;
  const size_t part_bytes = (plan.partial_bytes + 255) / 256 * 256;
  if (!a.scratch || (reinterpret_cast<uintptr_t>(a.scratch) & 255u) ||
      a.scratch_bytes < UNIQL_SCRATCH_COUNTER_BYTES + part_bytes)
    return UNIQL_ESCRATCH;
  p.counters = (int*)a.scratch;
  p.partials = (float*)((char*)a.scratch + UNIQL_SCRATCH_COUNTER_BYTES);
  const int grid_x = (p.nblk + p.WN - 1) / p.WN;
  if ((size_t)grid_x * sizeof(int) > UNIQL_SCRATCH_COUNTER_BYTES) return UNIQL_ESHAPE;
  if (a.comm) {
    p.cv = *a.comm;
    if (p.cv.reduce && (a.epilogue != UNIQL_EPILOGUE_NONE || a.nproj != 1)) return UNIQL_EINVAL;
    if (p.cv.reduce && vb > p.cv.block_cap) return UNIQL_ESHAPE;
    const int units = pair ? vb / 2 : vb;
    if (p.cv.gather_out && (p.cv.col_offset % 64 || p.cv.col_offset + (int64_t)units * 64 > p.cv.feat_cap)) return UNIQL_ESHAPE;
  }
  p.npf = 0;
  for (int i = 0; i < a.nprefetch && i < 4; ++i)
    if (a.prefetch_ptr[i] && a.prefetch_bytes[i] >= 128) {
      p.pf_ptr[p.npf] = (const unsigned char*)a.prefetch_ptr[i];
      p.pf_lines[p.npf] = (long long)(a.prefetch_bytes[i] / 128);
      ++p.npf;
    }
  dim3 grid(grid_x, p.S_split);

  auto kern = plan.MT == 1 ? w4a16_gemv_kernel<1> : w4a16_gemv_kernel<2>;
  {
    // function attributes are per device
    static thread_local bool attr_set[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev][plan.MT - 1]) {
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      attr_set[dev][plan.MT - 1] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  // Every launch may start early behind its predecessor; the kernel itself waits (griddepcontrol.wait)
  // before it touches anything another kernel could have written.
  static const int pdl_on = env_int("UNIQL_B200_PDL", 1);
  if (pdl_on) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (plan.cluster) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 1;
    attr[nattr].val.clusterDim.y = (unsigned)plan.S;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  UNIQL_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return UNIQL_OK;
}

}  // namespace uniql

extern "C" int uniql_w4a16_gemv_plan_check(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t* out5) {
  if (!n) return 1;
  return uniql::gemv_plan_check(m, k, n, nproj, epilogue, out5);
}
