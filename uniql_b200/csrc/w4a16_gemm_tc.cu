// Prefill-regime W4A16 linear (m > 16) for sm_100a: tcgen05 tensor cores with the accumulator in TMEM and the
// int4 -> fp16 dequantisation done on the SM in front of the MMA.  Two kernels:
//   w4a16_gemm_tc_kernel<H>      m > 128: activations are the 128-row operand, dequantised weights the N operand
//                                (shared memory);
//   w4a16_gemm_tc_swap_kernel    16 < m <= 128: operands swapped, dequantised weights written to tensor memory.
//
// Replaces the large-batch instantiations of UniQL's Marlin kernel (csrc/linear/marlin_gemm_kernel.cuh:176-740,
// tile table :802-810), which run mma.sync with dequantisation on the same warps, while consuming the same
// packed buffers (quantize/quantize_helpers.py:145-165 weight order, :54-62 scale order).
//
// w4a16_gemm_tc_kernel<H>.  Tile: (128 * H) batch rows x 256 output columns x 64 k per pipeline stage, one persistent
// CTA per SM.  H = 2 when the 256-row tiles still fill the GPU: the two 128-row halves are separate M=128 MMAs that
// read the same dequantised weight tile, which halves the dequantisation work and the shared-memory writes per
// tensor-core cycle; their accumulators are the two 256-column halves of TMEM.  H = 1 double-buffers one accumulator
// across tiles instead.
//   warp 0      TMA producer: activation tile(s) [128 x 64] fp16 (128B-swizzled, K-major); no multicast.
//   warp 1      allocates TMEM (2 x 256 fp32 columns); one elected lane issues, per stage, one block of
//               tcgen05.mma kind::f16 (M=128, N=256, K=16) + the commit that releases the stage + a poll of the next
//               stage's barrier whose latency hides behind the MMA issue.
//   warps 2..   epilogue (4 per 128-row half): tcgen05.ld (32 lanes x 32 columns), + bias, fp32 -> fp16, row-major
//               stores; with H = 1 it overlaps the next tile's main loop through the second TMEM accumulator.
//   16 warps    dequantise, as two sets of eight that convert alternate stages so two stages are always in
//               conversion: packed words straight from global memory into registers (requested two stages ahead,
//               no hop through shared memory), exact (q - 8) in fp16 via LOP3 + HSUB2/HFMA2, one HMUL2 by the group
//               scale (bit-identical to the reference's dequantised weight), 32-bit stores into the K-major
//               128B-swizzled B tile (bank-conflict free), fence.proxy.async, arrive.
// One barrier per stage collects both the TMA bytes of the activation tile and the arrivals of the dequantise warps, so
// the issuing thread pays one wait per stage.
// Roofline: tensor pipe (2*m*n*k flops); algorithmic bytes k*n/2 + (k/128)*n*2 + m*k*2 + m*n*2.
// Every mbarrier wait is bounded; a wait that gives up sets UNIQL_STATUS_WAIT_TIMEOUT and the kernel drains.
#include "common.cuh"
#include "linear_internal.cuh"
#include "tma.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

namespace uniql {

namespace tc {
constexpr int BMH = 128, BN = 256, BK = 64;   // BMH: rows of one MMA (one "half")
constexpr int A_BYTES = BMH * BK * 2;         // 16 KB per half
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int DEQ_SETS = 2;                   // dequantise warp sets; set t converts k-blocks t, t + 2, ...
constexpr int DEQ_SET_WARPS = 8;              // per set: 4 column blocks x 2 pairs of packed rows
constexpr int DEQ_WARPS = DEQ_SETS * DEQ_SET_WARPS;
constexpr int TMEM_COLS = 512;
template <int H> struct Cfg {
  static constexpr int AB_STAGES = H == 1 ? 4 : 3;
  static constexpr int STAGE_A = H * A_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + AB_STAGES * STAGE_A;
  static constexpr int OFF_BAR = OFF_B + AB_STAGES * B_BYTES;
  static constexpr int NUM_BARS = 2 * AB_STAGES + 4;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16 + 1024;   // + slack to align the base to 1 KB
  static constexpr int FIRST_EPI_WARP = 2;
  static constexpr int EPI_WARPS = 4 * H;
  static constexpr int FIRST_DEQ_WARP = FIRST_EPI_WARP + EPI_WARPS;
  static constexpr int THREADS = (FIRST_DEQ_WARP + DEQ_WARPS) * 32;
};
// instruction descriptor: D fp32, A/B fp16, both K-major, N = 256, M = 128
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BMH >> 4) << 24);
// A blocking wait is a loop of mbarrier.try_wait with a suspend-time hint: the hardware parks the thread until the
// phase completes or the hint runs out, so a waiting warp issues almost nothing (polling used to be half of all issued
// instructions of the prefill kernel).  The loop gives up after WAIT_POLLS tries: about two seconds.
#ifndef UNIQL_TC_WAIT_POLLS
#define UNIQL_TC_WAIT_POLLS (1 << 17)
#endif
#ifndef UNIQL_TC_WAIT_HINT_NS
#define UNIQL_TC_WAIT_HINT_NS 16384
#endif
constexpr int WAIT_POLLS = UNIQL_TC_WAIT_POLLS;
constexpr uint32_t WAIT_HINT_NS = UNIQL_TC_WAIT_HINT_NS;
}  // namespace tc

struct TcParams {
  const uint4* B;        // packed weights [K/16][2N] words
  const uint4* S;        // permuted scales, row g has n/8 uint4
  const __half* bias;
  __half* D;
  int64_t ldd;
  int M, N, n_out, K;
  int mtiles, ntiles;
  int* status_word;
};

__device__ __forceinline__ uint32_t tc_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < tc::WAIT_POLLS; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(tc::WAIT_HINT_NS)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart; descriptor version 1 (sm_100)
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 tc_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// Wait used by warps that sit idle for most of a tile (same parked wait; kept as a separate name for the call sites).
__device__ __forceinline__ bool tc_mbar_wait_relaxed(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < tc::WAIT_POLLS; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(tc::WAIT_HINT_NS)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One poll of two barriers at once, so that the two shared-memory round trips overlap: bit 0 / bit 1 of the result
// say which phase has completed.
__device__ __forceinline__ uint32_t tc_try_wait2(uint32_t bar_a, uint32_t par_a, uint32_t bar_b, uint32_t par_b) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred pa, pb;\n\t.reg .u32 ra, rb;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 pa, [%1], %2, %5;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 pb, [%3], %4, %5;\n\t"
      "selp.u32 ra, 1, 0, pa;\n\t"
      "selp.u32 rb, 2, 0, pb;\n\t"
      "or.b32 %0, ra, rb;\n\t}"
      : "=r"(ok)
      : "r"(bar_a), "r"(par_a), "r"(bar_b), "r"(par_b), "r"(tc::WAIT_HINT_NS)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool tc_wait2(uint32_t bar_a, uint32_t par_a, uint32_t bar_b, uint32_t par_b) {
  uint32_t done = 0;
  for (int it = 0; it < tc::WAIT_POLLS; ++it) {
    done |= tc_try_wait2(bar_a, par_a, bar_b, par_b);
    if (done == 3) return true;
  }
  return false;
}

// All MMAs of one 64-k stage (four K=16 steps for each 128-row half), the commit that releases the stage, and one poll
// of the NEXT stage's barrier, in one block: the poll is issued first and its result read last, so its latency hides
// behind the issue of the MMAs instead of adding to the single issuing thread's serial time per stage.  Returns
// whether the next stage was already full.
template <int H>
__device__ __forceinline__ uint32_t tc_issue_stage(uint32_t tmem_d, uint64_t adesc0, uint64_t adesc1, uint64_t bdesc,
                                                   uint32_t accumulate, uint32_t bar_release, uint32_t bar_next,
                                                   uint32_t par_next) {
  uint32_t ok;
  if (H == 1) {
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%7], %8;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "add.u64 a1, %2, 2;\n\tadd.u64 a2, %2, 4;\n\tadd.u64 a3, %2, 6;\n\t"
        "add.u64 b1, %3, 2;\n\tadd.u64 b2, %3, 4;\n\tadd.u64 b3, %3, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %4, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %4, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %4, t;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(ok)
        : "r"(tmem_d), "l"(adesc0), "l"(bdesc), "r"(tc::IDESC), "r"(accumulate), "r"(bar_release), "r"(bar_next),
          "r"(par_next)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t.reg .b64 a1, a2, a3, c1, c2, c3, b1, b2, b3;\n\t.reg .b32 d1;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%8], %9;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "add.u32 d1, %1, 256;\n\t"
        "add.u64 a1, %2, 2;\n\tadd.u64 a2, %2, 4;\n\tadd.u64 a3, %2, 6;\n\t"
        "add.u64 c1, %3, 2;\n\tadd.u64 c2, %3, 4;\n\tadd.u64 c3, %3, 6;\n\t"
        "add.u64 b1, %4, 2;\n\tadd.u64 b2, %4, 4;\n\tadd.u64 b3, %4, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %4, %5, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %5, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %5, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %5, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [d1], %3, %4, %5, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [d1], c1, b1, %5, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [d1], c2, b2, %5, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [d1], c3, b3, %5, t;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(ok)
        : "r"(tmem_d), "l"(adesc0), "l"(adesc1), "l"(bdesc), "r"(tc::IDESC), "r"(accumulate), "r"(bar_release),
          "r"(bar_next), "r"(par_next)
        : "memory");
  }
  return ok;
}

template <int H>
__global__ void __launch_bounds__(tc::Cfg<H>::THREADS, 1)
w4a16_gemm_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap amap) {
  using namespace tc;
  constexpr int AB_STAGES = Cfg<H>::AB_STAGES, STAGE_A = Cfg<H>::STAGE_A;
  constexpr int OFF_A = Cfg<H>::OFF_A, OFF_B = Cfg<H>::OFF_B, OFF_BAR = Cfg<H>::OFF_BAR;
  constexpr int NUM_BARS = Cfg<H>::NUM_BARS, FIRST_EPI_WARP = Cfg<H>::FIRST_EPI_WARP;
  constexpr int FIRST_DEQ_WARP = Cfg<H>::FIRST_DEQ_WARP;
  static_assert(BN == 256, "the second accumulator sits 256 tensor-memory columns after the first");
  extern __shared__ uint8_t smem_unaligned[];
  // 1 KB alignment: the 128B-swizzled tiles must start on a swizzle-atom boundary
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = tc_smem_addr(smem);
  const uint32_t bars = sbase + OFF_BAR;
  // full[s]: the activation tile has landed (TMA bytes) AND one set's warps have written the weight tile;
  // empty[s]: the MMAs that read stage s have completed
  const uint32_t bar_full = bars, bar_empty_ab = bars + 8 * AB_STAGES;
  const uint32_t bar_tmem_full = bars + 16 * AB_STAGES, bar_tmem_empty = bar_tmem_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / BK;
  const int total_tiles = p.mtiles * p.ntiles;
  const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total_it = my_tiles * KB;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&amap) : "memory");
    for (int s = 0; s < AB_STAGES; ++s) {
      tc_mbar_init(bar_full + 8 * s, 1 + DEQ_SET_WARPS);
      tc_mbar_init(bar_empty_ab + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(bar_tmem_full + 8 * b, 1);
      tc_mbar_init(bar_tmem_empty + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_addr((const void*)tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool timed_out = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      int it_ab = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int mt = tile % p.mtiles;
        for (int kb = 0; kb < KB; ++kb, ++it_ab) {
          const int s = it_ab % AB_STAGES;
          if (!timed_out && !tc_mbar_wait(bar_empty_ab + 8 * s, ((it_ab / AB_STAGES) & 1) ^ 1)) timed_out = true;
          tc_mbar_expect_tx(bar_full + 8 * s, STAGE_A);
#pragma unroll
          for (int h = 0; h < H; ++h)
            tc_tma_2d(sbase + OFF_A + s * STAGE_A + h * A_BYTES, &amap, kb * BK, (mt * H + h) * BMH, bar_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it_ab = 0, it_tile = 0;
      uint32_t ready = 0;                        // the current stage's full barrier was seen complete by the last poll
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it_tile) {
        // H == 1: one accumulator per tile, alternating between the two TMEM halves (epilogue of tile t overlaps
        // the main loop of tile t+1).  H == 2: both halves belong to this tile.
        const int buf0 = H == 1 ? (it_tile & 1) : 0;
        const uint32_t empty_parity = (H == 1 ? ((it_tile >> 1) & 1) : (it_tile & 1)) ^ 1;
#pragma unroll
        for (int h = 0; h < H; ++h)
          if (!timed_out && !tc_mbar_wait(bar_tmem_empty + 8 * (buf0 + h), empty_parity)) timed_out = true;
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb, ++it_ab) {
          const int s = it_ab % AB_STAGES;
          if (!ready && !timed_out && !tc_mbar_wait(bar_full + 8 * s, (it_ab / AB_STAGES) & 1)) timed_out = true;
          tc_fence_after();
          const int s1 = (s + 1 == AB_STAGES) ? 0 : s + 1;
          const uint64_t adesc0 = tc_smem_desc(sbase + OFF_A + s * STAGE_A);
          ready = tc_issue_stage<H>(tmem_base + buf0 * BN, adesc0, adesc0 + (A_BYTES >> 4),
                                    tc_smem_desc(sbase + OFF_B + s * B_BYTES), kb != 0 ? 1u : 0u, bar_empty_ab + 8 * s,
                                    bar_full + 8 * s1, ((it_ab + 1) / AB_STAGES) & 1);
          if (it_ab + 1 >= total_it) ready = 0;   // that poll looked at a phase nobody will complete
        }
#pragma unroll
        for (int h = 0; h < H; ++h) tc_commit(bar_tmem_full + 8 * (buf0 + h));   // accumulators complete
      }
    }
  } else if (warp < FIRST_DEQ_WARP) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;                     // TMEM lane quadrant this warp may access
    const int half = (warp - FIRST_EPI_WARP) >> 2;   // which 128-row half of the tile (always 0 when H == 1)
    int it_tile = 0;
    const bool vec_ok = ((p.ldd & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0);
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it_tile) {
      const int mt = tile % p.mtiles, nt = tile / p.mtiles;
      const int buf = H == 1 ? (it_tile & 1) : half;
      const uint32_t full_parity = H == 1 ? ((it_tile >> 1) & 1) : (it_tile & 1);
      if (!timed_out && !tc_mbar_wait_relaxed(bar_tmem_full + 8 * buf, full_parity)) timed_out = true;
      tc_fence_after();
      const int m = (mt * H + half) * BMH + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      __half* drow = p.D + (size_t)m * p.ldd;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc_ld32(taddr + c0, r);
        const int n0 = nt * BN + c0;
        if (m < p.M && n0 < p.n_out) {
          if (vec_ok && n0 + 32 <= p.n_out) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t pk[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float f0 = __uint_as_float(r[8 * v + 2 * e]), f1 = __uint_as_float(r[8 * v + 2 * e + 1]);
                if (p.bias) {
                  f0 += __half2float(p.bias[n0 + 8 * v + 2 * e]);
                  f1 += __half2float(p.bias[n0 + 8 * v + 2 * e + 1]);
                }
                __half2 h = __floats2half2_rn(f0, f1);
                pk[e] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(drow + n0 + 8 * v) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (n0 + e < p.n_out) {
                float f = __uint_as_float(r[e]);
                if (p.bias) f += __half2float(p.bias[n0 + e]);
                drow[n0 + e] = __float2half_rn(f);
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(bar_tmem_empty + 8 * buf);
    }
  } else {
    // ------------------------------------------------------------------ dequantise
    // Two sets of eight warps convert alternate k-blocks, so that two stages are in conversion at any time: what
    // bounds this path is the latency of one warp's chain per stage (barrier polls, packed-word read, convert, store,
    // proxy fence, arrive), not its instruction count.
    const int dw = warp - FIRST_DEQ_WARP;
    const int set = dw / DEQ_SET_WARPS;
    const int blk_local = dw & 3;               // 64-column block of the 256-column tile
    const int kt0 = ((dw >> 2) & 1) * 2;        // this warp's two packed rows of the stage: k = 16 kt0 .. 16 kt0 + 31
    const int g = lane >> 2, c = lane & 3;
    const int nblk = p.N >> 6;
    const uint32_t srow_u4 = (uint32_t)(p.N >> 3);
    const uint4* sbase_g = p.S + g;
    // position of the k-block this warp converts next, and of the one after it (whose scales are requested early)
    int ti = 0, kb = set;
    while (kb >= KB && ti < my_tiles) { kb -= KB; ++ti; }
    int ti2 = ti, kb2 = kb + DEQ_SETS;
    while (kb2 >= KB && ti2 < my_tiles) { kb2 -= KB; ++ti2; }
    // The packed words come straight from global memory into registers (512 contiguous bytes per warp and packed
    // row), requested one iteration = two k-blocks ahead like the scales: a hop through shared memory would add a
    // barrier wait and a read to the chain that bounds this path, and 16 KB per stage to the shared-memory traffic.
    const uint32_t prow_u4 = (uint32_t)(p.N >> 1);            // one packed row: 2N words = N/2 uint4
    const uint4* pbase = p.B + (size_t)kt0 * prow_u4 + lane;
    const uint4 kZero = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // (8 - 8) * scale = 0
    uint4 snext = make_uint4(0, 0, 0, 0), wnext[2] = {kZero, kZero};
    if (set < total_it) {
      const int blk = (((int)blockIdx.x + ti * (int)gridDim.x) / p.mtiles) * 4 + blk_local;
      if (blk < nblk) {
        snext = ld_nc16(sbase_g + (size_t)blk * 8 + (size_t)(kb >> 1) * srow_u4);
        const uint4* src = pbase + (size_t)kb * 4 * prow_u4 + (size_t)blk * 32;
        wnext[0] = ld_nc16(src);
        wnext[1] = ld_nc16(src + prow_u4);
      }
    }
    for (int it = set; it < total_it; it += DEQ_SETS) {
      uint32_t sdup[8];                         // the lane's 8 group scales, each duplicated into a half2
      const uint4 w4[2] = {wnext[0], wnext[1]};
      {
        const uint32_t s4[4] = {snext.x, snext.y, snext.z, snext.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sdup[2 * j] = __byte_perm(s4[j], 0, 0x1010);       // low half  -> columns 16j+g
          sdup[2 * j + 1] = __byte_perm(s4[j], 0, 0x3232);   // high half -> columns 16j+g+8
        }
        if (it + DEQ_SETS < total_it) {
          const int blk2 = (((int)blockIdx.x + ti2 * (int)gridDim.x) / p.mtiles) * 4 + blk_local;
          wnext[0] = wnext[1] = kZero;
          if (blk2 < nblk) {
            snext = ld_nc16(sbase_g + (size_t)blk2 * 8 + (size_t)(kb2 >> 1) * srow_u4);
            const uint4* src = pbase + (size_t)kb2 * 4 * prow_u4 + (size_t)blk2 * 32;
            wnext[0] = ld_nc16(src);
            wnext[1] = ld_nc16(src + prow_u4);
          }
        }
        ti = ti2; kb = kb2;
        kb2 += DEQ_SETS;
        while (kb2 >= KB && ti2 < my_tiles) { kb2 -= KB; ++ti2; }
      }
      const int s = it % AB_STAGES;
      if (!timed_out && !tc_mbar_wait(bar_empty_ab + 8 * s, ((it / AB_STAGES) & 1) ^ 1)) timed_out = true;
      const uint32_t btile = sbase + OFF_B + s * B_BYTES + (uint32_t)(blk_local * 64 + g) * 128 + 4 * c;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int kt = kt0 + u;
        const uint32_t wq[4] = {w4[u].x, w4[u].y, w4[u].z, w4[u].w};
        const uint32_t a_lo = btile + ((uint32_t)((2 * kt) ^ g) << 4), a_hi = btile + ((uint32_t)((2 * kt + 1) ^ g) << 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t qw = wq[j], qs = wq[j] >> 8;
          uint32_t v;
          __half2 r;
          v = nib_pair_to_half2_m8(qw);                               // n = 16j+g,   k = 2c, 2c+1
          r = __hmul2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&sdup[2 * j]));
          tc_sts32(a_lo + (16 * j) * 128, *reinterpret_cast<uint32_t*>(&r));
          v = nib_pair_hi_to_half2_m8(qw);                            // n = 16j+g,   k = 2c+8, 2c+9
          r = __hmul2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&sdup[2 * j]));
          tc_sts32(a_hi + (16 * j) * 128, *reinterpret_cast<uint32_t*>(&r));
          v = nib_pair_to_half2_m8(qs);                               // n = 16j+g+8, k = 2c, 2c+1
          r = __hmul2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&sdup[2 * j + 1]));
          tc_sts32(a_lo + (16 * j + 8) * 128, *reinterpret_cast<uint32_t*>(&r));
          v = nib_pair_hi_to_half2_m8(qs);                            // n = 16j+g+8, k = 2c+8, 2c+9
          r = __hmul2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&sdup[2 * j + 1]));
          tc_sts32(a_hi + (16 * j + 8) * 128, *reinterpret_cast<uint32_t*>(&r));
        }
      }
      // make the generic-proxy stores visible to the tensor core's async-proxy reads, then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(bar_full + 8 * s);
    }
  }

  if (timed_out && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------------------
// Small-batch variant (16 < m <= 128): operands swapped.  The dequantised weight tile [128 columns x 128 k] is the
// 128-row MMA operand (tensor-memory lane = output column), the activation tile [Mb x 128 k] (Mb = m rounded up to 16)
// the N operand, so the MMA is 128 x Mb x 16 and no tensor work is spent on padding rows.  The weight operand never
// enters shared memory: the dequantise warps (four sets of four, one warp per 32-lane quarter of tensor memory, each
// set converting every fourth stage) write it to tensor memory with tcgen05.st and the MMA reads it from there, which
// removes the shared stores, the proxy fence and the tensor core's operand reads of it.  Only the packed words (8 KB
// per stage, TMA) and the activation tile (two swizzled [Mb x 64 k] sub-tiles, TMA) cross shared memory.
// What bounds this kernel is the latency of the hand-offs between the warp roles, paid once per stage: hence one scale
// group (128 k, eight MMAs) per stage, one merged barrier per stage, and the next-stage poll fused with the MMA issue.
// The accumulator holds D^T: the epilogue stores, per batch row, 32 adjacent columns per warp (64-byte segments).
// With few column tiles a cluster of up to 8 CTAs shares each tile, every CTA reducing a slice of k; the partial
// accumulators are summed in rank order through distributed shared memory (deterministic, no global scratch).
namespace tcs {
constexpr int BNW = 128, BK = 128;              // one stage = one scale group: the hand-offs between the warp roles,
                                                // which bound this kernel, are paid once per 128 k
constexpr int P_BYTES = (BK / 16) * (2 * BNW) * 4;   // 8 KB: 8 packed rows x 256 words
constexpr int STAGES = 4, P_STAGES = 8;
constexpr int NSETS = 4;                        // dequantise warp sets; set t converts k-blocks t, t + NSETS, ...
constexpr int DEQ_WARPS = 4;                    // warps per set: one per 32-lane quarter of tensor memory
constexpr int FIRST_DEQ_WARP = 7;
constexpr int OFF_P = 0;
constexpr int OFF_BAR = OFF_P + P_STAGES * P_BYTES;
constexpr int NUM_BARS = 2 * STAGES + 2 * P_STAGES + 4;
constexpr int OFF_X = OFF_BAR + 1024;           // activation ring: STAGES stages of two [Mb x 64 k] swizzled sub-tiles
constexpr int THREADS = (FIRST_DEQ_WARP + NSETS * DEQ_WARPS) * 32;
constexpr int TMEM_COLS = 512;                  // two accumulators of up to 128 columns, then the weight-tile ring
constexpr int TMEM_W0 = 256;                    // weight tile of stage s: columns TMEM_W0 + 64 s (128 k as 64 half2 columns)
static_assert(TMEM_W0 + STAGES * (BK / 2) <= TMEM_COLS, "tensor memory budget");
static_assert(NUM_BARS * 8 + 16 <= 1024, "barrier block");
static_assert(THREADS <= 1024, "block size");
// at least 120 KB, so that two CTAs (each allocates all 512 tensor-memory columns) can never share an SM
inline int smem_bytes(int Mb) {
  const int need = OFF_X + STAGES * Mb * (BK * 2) + 1024;
  return need < 120 * 1024 ? 120 * 1024 : need;
}
}  // namespace tcs

// Up to kMaxProj projections that read the same activations share one launch: their 128-column tiles form one list
// (q/k/v, or gate and up, of a decoder block at batches of 17..128 rows).
struct TcSwapProj {
  const uint4* S;
  const __half* bias;
  __half* D;
  int64_t ldd;
  int N, n_out;
};
struct TcSwapParams {
  TcSwapProj proj[kMaxProj];
  int tile_start[kMaxProj + 1];                 // first tile of each projection in the launch's tile list
  int nproj;
  int M, Mb, K;
  int ntiles;
  int split;                                    // CTAs of a cluster that share one column tile, each a slice of k
  int* status_word;
};
struct TcSwapMaps {
  CUtensorMap w[kMaxProj];                      // packed weights of each projection
};

// tile of the launch -> (projection, tile inside it)
__device__ __forceinline__ void tcs_proj_of(const TcSwapParams& p, int nt, int& pi, int& lt) {
  pi = 0;
#pragma unroll
  for (int i = 1; i < kMaxProj; ++i)
    if (i < p.nproj && nt >= p.tile_start[i]) pi = i;
  lt = nt - p.tile_start[pi];
}

__device__ __forceinline__ void tcs_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The eight MMAs of one 128-k stage, the commit that releases the stage, and one poll of the NEXT stage's barrier, in
// one block: the poll is issued first and its result read last, so its latency hides behind the issue of the MMAs
// instead of adding to the single issuing thread's serial time per stage.  The weight operand comes from tensor memory
// (8 columns per K=16 step), the activation operand from two swizzled [Mb x 64 k] sub-tiles in shared memory.
// Returns whether the next stage was already full.
__device__ __forceinline__ uint32_t tcs_issue_stage(uint32_t tmem_d, uint32_t tmem_w, uint64_t xdesc0, uint64_t xdesc1,
                                                    uint32_t idesc, uint32_t accumulate, uint32_t bar_release,
                                                    uint32_t bar_next, uint32_t par_next) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q, t;\n\t.reg .b32 a1, a2, a3, a4, a5, a6, a7;\n\t.reg .b64 b1, b2, b3, c1, c2, c3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%8], %9;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 a1, %2, 8;\n\tadd.u32 a2, %2, 16;\n\tadd.u32 a3, %2, 24;\n\tadd.u32 a4, %2, 32;\n\t"
      "add.u32 a5, %2, 40;\n\tadd.u32 a6, %2, 48;\n\tadd.u32 a7, %2, 56;\n\t"
      "add.u64 b1, %3, 2;\n\tadd.u64 b2, %3, 4;\n\tadd.u64 b3, %3, 6;\n\t"
      "add.u64 c1, %4, 2;\n\tadd.u64 c2, %4, 4;\n\tadd.u64 c3, %4, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], b1, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], b2, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], b3, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a4], %4, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a5], c1, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a6], c2, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a7], c3, %5, t;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(ok)
      : "r"(tmem_d), "r"(tmem_w), "l"(xdesc0), "l"(xdesc1), "r"(idesc), "r"(accumulate), "r"(bar_release),
        "r"(bar_next), "r"(par_next)
      : "memory");
  return ok;
}

__global__ void __launch_bounds__(tcs::THREADS, 1)
w4a16_gemm_tc_swap_kernel(const __grid_constant__ TcSwapParams p, const __grid_constant__ CUtensorMap xmap,
                          const __grid_constant__ TcSwapMaps wmaps) {
  using namespace tcs;
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = tc_smem_addr(smem);
  const uint32_t bars = sbase + OFF_BAR;
  // full[s]: the activation tile has landed in shared memory (TMA bytes) AND the set's warps have written the weight
  // tile of the stage into tensor memory;
  // empty[s]: the MMAs that read stage s have completed
  const uint32_t bar_full = bars, bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_full_p = bar_empty + 8 * STAGES, bar_empty_p = bar_full_p + 8 * P_STAGES;
  const uint32_t bar_tmem_full = bar_empty_p + 8 * P_STAGES, bar_tmem_empty = bar_tmem_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + NUM_BARS * 8);
  const uint32_t x_half = (uint32_t)p.Mb * 128;   // one [Mb x 64 k] sub-tile
  const uint32_t x_bytes = 2 * x_half;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a cluster of p.split CTAs owns one column tile at a time; CTA `rank` of it reduces k-blocks (= scale groups)
  // [kb0, kb0 + KB)
  const int rank = (int)blockIdx.x % p.split;
  const int tile0 = (int)blockIdx.x / p.split, tile_step = (int)gridDim.x / p.split;
  const int groups = p.K / 128;
  const int kb0 = (int)((long long)groups * rank / p.split);
  const int KB = (int)((long long)groups * (rank + 1) / p.split) - kb0;
  const int my_tiles = (tile0 < p.ntiles) ? (p.ntiles - 1 - tile0) / tile_step + 1 : 0;
  const int total_it = my_tiles * KB;
  // instruction descriptor: D fp32, A/B fp16, both K-major, M = 128 (weight columns), N = Mb (batch rows)
  const uint32_t idesc = (1u << 4) | ((uint32_t)(p.Mb >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

  pdl_launch_dependents();                       // the next kernel in the stream may start its own set-up and weights
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
    for (int i = 0; i < p.nproj; ++i) asm volatile("prefetch.tensormap [%0];" ::"l"(&wmaps.w[i]) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(bar_full + 8 * s, 1 + DEQ_WARPS);
      tc_mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < P_STAGES; ++s) {
      tc_mbar_init(bar_full_p + 8 * s, 1);
      tc_mbar_init(bar_empty_p + 8 * s, DEQ_WARPS);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(bar_tmem_full + 8 * b, 1);
      tc_mbar_init(bar_tmem_empty + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_addr((const void*)tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool timed_out = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ packed-weight producer (the HBM stream)
    if (lane == 0) {
      int it = 0;
      for (int nt = tile0; nt < p.ntiles; nt += tile_step) {
        int pi, lt;
        tcs_proj_of(p, nt, pi, lt);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int sp = it % P_STAGES;
          if (!timed_out && !tc_mbar_wait(bar_empty_p + 8 * sp, ((it / P_STAGES) & 1) ^ 1)) timed_out = true;
          tc_mbar_expect_tx(bar_full_p + 8 * sp, P_BYTES);
          tc_tma_2d(sbase + OFF_P + sp * P_BYTES, &wmaps.w[pi], lt * (2 * BNW), (kb0 + kb) * (BK / 16), bar_full_p + 8 * sp);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ activation producer (re-reads, L2 hits)
    if (lane == 0) {
      // Programmatic dependent launch: everything up to here (barriers, tensor memory, the first weight tiles, the
      // dequantise warps' scale loads) ran while the producer of the activations was still finishing; the activation
      // tiles are the only thing that has to wait for it.  Results are stored after MMAs that consumed those tiles.
      pdl_wait();
      int kb = 0;
      for (int it = 0; it < total_it; ++it) {
        const int s = it % STAGES;
        if (!timed_out && !tc_mbar_wait(bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1)) timed_out = true;
        tc_mbar_expect_tx(bar_full + 8 * s, x_bytes);
        tc_tma_2d(sbase + OFF_X + s * x_bytes, &xmap, (kb0 + kb) * BK, 0, bar_full + 8 * s);
        tc_tma_2d(sbase + OFF_X + s * x_bytes + x_half, &xmap, (kb0 + kb) * BK + 64, 0, bar_full + 8 * s);
        if (++kb == KB) kb = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it = 0, it_tile = 0;
      uint32_t ready = 0;                        // the current stage's full barrier was seen complete by the last poll
      for (int nt = tile0; nt < p.ntiles; nt += tile_step, ++it_tile) {
        const int buf = it_tile & 1;
        if (!timed_out && !tc_mbar_wait(bar_tmem_empty + 8 * buf, ((it_tile >> 1) & 1) ^ 1)) timed_out = true;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 128;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ready && !timed_out && !tc_mbar_wait(bar_full + 8 * s, (it / STAGES) & 1)) timed_out = true;
          tc_fence_after();
          const int s1 = (s + 1 == STAGES) ? 0 : s + 1;
          ready = tcs_issue_stage(tmem_d, tmem_base + TMEM_W0 + s * (BK / 2), tc_smem_desc(sbase + OFF_X + s * x_bytes),
                                  tc_smem_desc(sbase + OFF_X + s * x_bytes + x_half), idesc, kb != 0 ? 1u : 0u,
                                  bar_empty + 8 * s, bar_full + 8 * s1, ((it + 1) / STAGES) & 1);
          if (it + 1 >= total_it) ready = 0;      // that poll looked at a phase nobody will complete
        }
        tc_commit(bar_tmem_full + 8 * buf);
      }
    }
  } else if (warp < FIRST_DEQ_WARP) {
    // ------------------------------------------------------------------ epilogue (D^T: lane = column, TMEM column = batch row)
    const int q = warp & 3;
    int it_tile = 0;
    if (p.split > 1) {
      // one tile per cluster: every rank parks its partial accumulator in shared memory (the activation ring, idle
      // once the last MMA has completed) as part[batch row][column]; after the cluster barrier every rank sums a slice
      // of the batch rows over all ranks
      if (tile0 < p.ntiles) {
        if (!timed_out && !tc_mbar_wait_relaxed(bar_tmem_full, 0)) timed_out = true;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t part = sbase + OFF_X + (uint32_t)(q * 32 + lane) * 4;
#pragma unroll 1
        for (int c0 = 0; c0 < p.Mb; c0 += 32) {
          uint32_t r[32];
          tc_ld32(taddr + c0, r);
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c0 + e < p.M) tc_sts32(part + (uint32_t)(c0 + e) * (BNW * 4), r[e]);
        }
      }
    } else
    for (int nt = tile0; nt < p.ntiles; nt += tile_step, ++it_tile) {
      const int buf = it_tile & 1;
      if (!timed_out && !tc_mbar_wait_relaxed(bar_tmem_full + 8 * buf, (it_tile >> 1) & 1)) timed_out = true;
      tc_fence_after();
      int pi, lt;
      tcs_proj_of(p, nt, pi, lt);
      const TcSwapProj& pr = p.proj[pi];
      const int n = lt * BNW + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 128;
      const float bv = (pr.bias && n < pr.n_out) ? __half2float(pr.bias[n]) : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < p.Mb; c0 += 32) {
        uint32_t r[32];
        tc_ld32(taddr + c0, r);
        if (n < pr.n_out) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c0 + e < p.M) pr.D[(size_t)(c0 + e) * pr.ldd + n] = __float2half_rn(__uint_as_float(r[e]) + bv);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(bar_tmem_empty + 8 * buf);
    }
  } else {
    // ------------------------------------------------------------------ dequantise into tensor memory
    // A lane of the Marlin layout holds, per packed word j, the half2 pairs (n = 16j+g | 16j+g+8) x (k = 2c.. | 2c+8..):
    // exactly the register fragment of tcgen05.st.16x128b (register 2i -> lane g, column 4i+c; 2i+1 -> lane g+8), so
    // the weight tile goes from registers to the MMA's A operand without touching shared memory.  Warp quarter q owns
    // tensor-memory lanes 32q..32q+31 = columns 32q.. of the tile = Marlin block q/2, words j = 2(q%2), 2(q%2)+1.
    const int dw = warp - FIRST_DEQ_WARP;
    const int set = dw / DEQ_WARPS;
    const int q = warp & 3;
    const int blk_local = q >> 1;
    const int g = lane >> 2;
    // scales of 64-column block `blk_local` of tile `nt` and k-block `kblk` (zero for a block past the projection's width)
    // (the projection of a tile is looked up when the tile changes, not per stage: this loop is latency-critical)
    int c_nt = -1, c_lt = 0, c_N = 0;
    const uint4* c_S = nullptr;
    auto load_scales = [&](int nt, int kblk, bool& valid) {
      if (nt != c_nt) {
        int pi, lt;
        tcs_proj_of(p, nt, pi, lt);
        c_nt = nt; c_lt = lt; c_N = p.proj[pi].N; c_S = p.proj[pi].S;
      }
      const int blk = c_lt * 2 + blk_local;
      valid = blk < (c_N >> 6);
      if (!valid) return make_uint2(0, 0);
      return __ldg(reinterpret_cast<const uint2*>(c_S + g + (size_t)blk * 8 + (size_t)kblk * (size_t)(c_N >> 3)) + (q & 1));
    };
    // position of the k-block this warp converts next, and of the one after it (whose scales are requested early)
    int ti = 0, kb = set;
    while (kb >= KB && ti < my_tiles) { kb -= KB; ++ti; }
    int ti2 = ti, kb2 = kb + NSETS;
    while (kb2 >= KB && ti2 < my_tiles) { kb2 -= KB; ++ti2; }
    uint2 snext = make_uint2(0, 0);
    bool vnext = false;
    if (set < total_it) snext = load_scales(tile0 + ti * tile_step, kb0 + kb, vnext);
    for (int it = set; it < total_it; it += NSETS) {
      const bool valid = vnext;
      uint32_t sdup[4];
      sdup[0] = __byte_perm(snext.x, 0, 0x1010);   // word j0:   columns 16 j0 + g
      sdup[1] = __byte_perm(snext.x, 0, 0x3232);   //            columns 16 j0 + g + 8
      sdup[2] = __byte_perm(snext.y, 0, 0x1010);   // word j0+1
      sdup[3] = __byte_perm(snext.y, 0, 0x3232);
      if (it + NSETS < total_it) snext = load_scales(tile0 + ti2 * tile_step, kb0 + kb2, vnext);
      ti = ti2; kb = kb2;
      kb2 += NSETS;
      while (kb2 >= KB && ti2 < my_tiles) { kb2 -= KB; ++ti2; }

      const int sp = it % P_STAGES, s = it % STAGES;
      if (!timed_out && !tc_wait2(bar_full_p + 8 * sp, (it / P_STAGES) & 1, bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1))
        timed_out = true;
      tc_fence_after();
      const uint32_t pk = sbase + OFF_P + sp * P_BYTES + blk_local * 512 + lane * 16 + (q & 1) * 8;
#pragma unroll
      for (int hk = 0; hk < 2; ++hk) {            // the two 64-k halves of the stage: packed rows 4 hk .. 4 hk + 3
        uint32_t wq[4][2];
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
          wq[kt][0] = wq[kt][1] = 0x88888888u;
          if (valid)
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];"
                         : "=r"(wq[kt][0]), "=r"(wq[kt][1]) : "r"(pk + (4 * hk + kt) * 1024) : "memory");
        }
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          uint32_t r[16];
          const __half2 s_lo = *reinterpret_cast<const __half2*>(&sdup[2 * jj]);
          const __half2 s_hi = *reinterpret_cast<const __half2*>(&sdup[2 * jj + 1]);
#pragma unroll
          for (int kt = 0; kt < 4; ++kt) {
            const uint32_t qw = wq[kt][jj], qs = qw >> 8;
            uint32_t v;
            __half2 h;
            v = nib_pair_to_half2_m8(qw);                               // n = 16j+g,   k = 16kt + 2c, 2c+1
            h = __hmul2(*reinterpret_cast<__half2*>(&v), s_lo);
            r[4 * kt + 0] = *reinterpret_cast<uint32_t*>(&h);
            v = nib_pair_to_half2_m8(qs);                               // n = 16j+g+8, k = 16kt + 2c, 2c+1
            h = __hmul2(*reinterpret_cast<__half2*>(&v), s_hi);
            r[4 * kt + 1] = *reinterpret_cast<uint32_t*>(&h);
            v = nib_pair_hi_to_half2_m8(qw);                            // n = 16j+g,   k = 16kt + 2c+8, 2c+9
            h = __hmul2(*reinterpret_cast<__half2*>(&v), s_lo);
            r[4 * kt + 2] = *reinterpret_cast<uint32_t*>(&h);
            v = nib_pair_hi_to_half2_m8(qs);                            // n = 16j+g+8, k = 16kt + 2c+8, 2c+9
            h = __hmul2(*reinterpret_cast<__half2*>(&v), s_hi);
            r[4 * kt + 3] = *reinterpret_cast<uint32_t*>(&h);
          }
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32 + jj * 16) << 16) + TMEM_W0 + s * (BK / 2) + hk * 32;
          asm volatile(
              "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "
              "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
              ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
              : "memory");
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        tc_mbar_arrive(bar_full + 8 * s);
        tc_mbar_arrive(bar_empty_p + 8 * sp);
      }
    }
  }

  if (p.split > 1) {
    __syncwarp();
    tcs_cluster_sync();                         // every rank's partial is in its shared memory
    if (warp >= 3 && tile0 < p.ntiles) {
      // Rank r finishes batch rows [Mb r / split, Mb (r+1) / split).  All twenty warps past the producers take part (the
      // dequantise warps are idle by now): four warps cover the 128 columns, five such groups interleave the rows, so a
      // thread has at most four rows x `split` partials to fetch -- all of them independent loads from the ranks'
      // shared memory (distributed shared memory), in flight together, added in rank order so that the sum does not
      // depend on timing.  (With rank 0's four warps alone walking the peers one after the other this step took 6 us
      // at split 4 and 14 us at split 8: every batch of remote loads is a ~1 us round trip.)
      const int q = (warp - 3) & 3, grp = (warp - 3) >> 2;
      int pi, lt;
      tcs_proj_of(p, tile0, pi, lt);
      const TcSwapProj& pr = p.proj[pi];
      const int n = lt * BNW + q * 32 + lane;
      const uint32_t part = sbase + OFF_X + (uint32_t)(q * 32 + lane) * 4;
      const float bv = (pr.bias && n < pr.n_out) ? __half2float(pr.bias[n]) : 0.f;
      uint32_t remote[8];
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        remote[rr] = part;
        if (rr < p.split) asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[rr]) : "r"(part), "r"(rr));
      }
      const int row0 = p.Mb * rank / p.split;
      int row1 = p.Mb * (rank + 1) / p.split;
      if (row1 > p.M) row1 = p.M;
#pragma unroll 1
      for (int r0 = row0 + grp; r0 < row1; r0 += 20) {
        float v[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            v[i][rr] = 0.f;
            if (rr < p.split && r0 + 5 * i < row1)
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[i][rr]) : "r"(remote[rr] + (uint32_t)(r0 + 5 * i) * (BNW * 4)));
          }
        if (n < pr.n_out) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (r0 + 5 * i < row1) {
              float acc = v[i][0];
#pragma unroll
              for (int rr = 1; rr < 8; ++rr)
                if (rr < p.split) acc += v[i][rr];
              pr.D[(size_t)(r0 + 5 * i) * pr.ldd + n] = __float2half_rn(acc + bv);
            }
        }
      }
    }
    __syncwarp();
    tcs_cluster_sync();                         // no rank leaves while its shared memory may still be read
  }
  if (timed_out && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
static EncodeTiledFn tc_encode_fn() { return encode_tiled_fn(); }   // shared, initialised once (thread-safe)

bool gemm_tc_supported(int64_t m, int64_t n, int64_t k) {
  return m > 16 && n >= 128 && n % 64 == 0 && k % 128 == 0;
}

size_t gemm_tc_scratch_bytes(int64_t, int64_t, int64_t) { return 0; }

// Clusters of `split` CTAs of the small-batch kernel that can be resident together (0 if the query fails).
static int max_active_clusters(int split, int smem) {
  static thread_local int cache[64][9][2];      // [device][split] -> {smem the answer is for, answer}; per thread: no races
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || split < 1 || split > 8) return 0;
  if (cache[dev][split][0] == smem) return cache[dev][split][1];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(split * 64));
  cfg.blockDim = dim3(tcs::THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, w4a16_gemm_tc_swap_kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  cache[dev][split][0] = smem;
  cache[dev][split][1] = n;
  return n;
}

// Projections of one launch (same activations, same k); D[i] receives projection i.
static int launch_gemm_tc_swap(const LinearArgs* projs, void* const* Ds, int nproj, const __half* A, int64_t lda,
                               int64_t m, cudaStream_t stream) {
  using namespace tcs;
  if (nproj < 1 || nproj > kMaxProj) return UNIQL_EINVAL;
  const LinearArgs& a = projs[0];
  EncodeTiledFn enc = tc_encode_fn();
  if (!enc) return cuda_fail(cudaErrorNotSupported);
  const int Mb = (int)((m + 15) / 16 * 16);
  CUtensorMap xmap;
  TcSwapMaps wmaps;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)Mb};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(A), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cuda_fail(cudaErrorInvalidValue);
  }
  TcSwapParams p;
  memset(&p, 0, sizeof(p));
  int tiles = 0;
  for (int i = 0; i < nproj; ++i) {
    const LinearArgs& q = projs[i];
    if (q.k != a.k || q.n < 128 || q.n % 64) return UNIQL_ESHAPE;
    cuuint64_t dims[2] = {(cuuint64_t)(2 * q.n), (cuuint64_t)(q.k / 16)};
    cuuint64_t strides[1] = {(cuuint64_t)(2 * q.n) * 4};
    cuuint32_t box[2] = {256, (cuuint32_t)(BK / 16)};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&wmaps.w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(q.B), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cuda_fail(cudaErrorInvalidValue);
    p.proj[i].S = (const uint4*)q.s; p.proj[i].bias = (const __half*)q.bias; p.proj[i].D = (__half*)Ds[i];
    p.proj[i].ldd = q.ldd; p.proj[i].N = (int)q.n; p.proj[i].n_out = (int)q.n_out;
    p.tile_start[i] = tiles;
    tiles += (int)((q.n + BNW - 1) / BNW);
  }
  for (int i = nproj; i <= kMaxProj; ++i) p.tile_start[i] = tiles;
  for (int i = nproj; i < kMaxProj; ++i) { wmaps.w[i] = wmaps.w[0]; p.proj[i] = p.proj[0]; }
  p.nproj = nproj;
  p.M = (int)m; p.Mb = Mb; p.K = (int)a.k;
  p.ntiles = tiles;
  p.status_word = a.status_word;
  {
    // function attributes are per device
    static thread_local bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(w4a16_gemm_tc_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          smem_bytes(128)));
      attr_set[dev] = true;
    }
  }
  const int sms = device_info().sm_count;
  // few column tiles: a cluster of `split` CTAs shares each tile, every CTA reducing a slice of k (at least four
  // scale groups), and the partial accumulators are summed through distributed shared memory
  int split = 1;
  {
    static const int forced = [] { const char* e = getenv("UNIQL_B200_TC_SPLIT"); return (e && *e) ? atoi(e) : 0; }();
    const int groups = (int)(a.k / 128);
    if (forced > 0) split = forced;
    else if (p.ntiles * 2 <= sms) {
      split = sms / p.ntiles;
      if (split > 8) split = 8;
      while (split > 1 && groups / split < 4) --split;
    }
    if (split > groups) split = groups;
    if (split < 1) split = 1;
    if (split > 8) split = 8;
    // every cluster must be resident at once (a second wave would cost more than the split gains): clusters are
    // placed inside one GPC, so fewer fit than SMs / split suggests
    while (split > 1 && forced <= 0 && max_active_clusters(split, smem_bytes(Mb)) < p.ntiles) --split;
  }
  p.split = split;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = split == 1 ? dim3((unsigned)(p.ntiles < sms ? p.ntiles : sms)) : dim3((unsigned)(p.ntiles * split));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = (size_t)smem_bytes(Mb);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  // may start behind its predecessor; the kernel waits (griddepcontrol.wait) before it reads the activations
  static const bool pdl_on = [] { const char* e = getenv("UNIQL_B200_PDL"); return !(e && *e && atoi(e) == 0); }();
  if (pdl_on) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (split > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = (unsigned)split;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  UNIQL_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a16_gemm_tc_swap_kernel, p, xmap, wmaps));
  return launch_status();
}

bool gemm_tc_group_supported(int64_t m, int64_t k, const int64_t* n, int nproj) {
  static const int swap_on = [] { const char* e = getenv("UNIQL_B200_TC_SWAP"); return (e && *e) ? atoi(e) : 1; }();
  if (!swap_on || m <= 16 || m > 128 || k % 128 || nproj < 1 || nproj > kMaxProj) return false;
  for (int i = 0; i < nproj; ++i)
    if (n[i] < 128 || n[i] % 64) return false;
  return true;
}

int launch_gemm_tc_group(const LinearArgs* projs, void* const* Ds, int nproj, const __half* A, int64_t lda, int64_t m,
                         cudaStream_t stream) {
  return launch_gemm_tc_swap(projs, Ds, nproj, A, lda, m, stream);
}

int launch_gemm_tc(const LinearArgs& a, const __half* A, int64_t lda, __half* D, int64_t m, cudaStream_t stream) {
  using namespace tc;
  static const int swap_on = [] { const char* e = getenv("UNIQL_B200_TC_SWAP"); return (e && *e) ? atoi(e) : 1; }();
  if (swap_on && m <= 128) {
    void* d1[1] = {D};
    return launch_gemm_tc_swap(&a, d1, 1, A, lda, m, stream);
  }
  EncodeTiledFn enc = tc_encode_fn();
  if (!enc) return cuda_fail(cudaErrorNotSupported);
  CUtensorMap amap;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BMH};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(A), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cuda_fail(cudaErrorInvalidValue);
  }
  TcParams p;
  p.B = (const uint4*)a.B; p.S = (const uint4*)a.s; p.bias = (const __half*)a.bias; p.D = D; p.ldd = a.ldd;
  p.M = (int)m; p.N = (int)a.n; p.n_out = (int)a.n_out; p.K = (int)a.k;
  // 256-row tiles share each dequantised weight tile between two MMAs; use them once they still fill the GPU
  p.ntiles = (int)((a.n + BN - 1) / BN);
  const int sms_ = device_info().sm_count;
  const int H = (m > BMH && ((m + 2 * BMH - 1) / (2 * BMH)) * (int64_t)p.ntiles >= sms_) ? 2 : 1;
  p.mtiles = (int)((m + H * BMH - 1) / (H * BMH));
  p.status_word = a.status_word;
  {
    static thread_local bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(w4a16_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          Cfg<1>::SMEM_BYTES));
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(w4a16_gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          Cfg<2>::SMEM_BYTES));
      attr_set[dev] = true;
    }
  }
  const int64_t tiles = (int64_t)p.mtiles * p.ntiles;
  const int sms = device_info().sm_count;
  const int grid = (int)(tiles < sms ? tiles : sms);
  if (H == 1)
    w4a16_gemm_tc_kernel<1><<<grid, Cfg<1>::THREADS, Cfg<1>::SMEM_BYTES, stream>>>(p, amap);
  else
    w4a16_gemm_tc_kernel<2><<<grid, Cfg<2>::THREADS, Cfg<2>::SMEM_BYTES, stream>>>(p, amap);
  return launch_status();
}

}  // namespace uniql
