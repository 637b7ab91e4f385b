// mbarrier / TMA helpers shared by the decode kernels (sm_100a).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace uniql {

constexpr int kSlotBytes = 4096;   // one quantisation group (8 packed rows) of one 64-column block

// ---- mbarrier / TMA helpers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: gives up after ~2^20 polls and reports it instead of hanging.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 20); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// One 2-D tile (128 words x 8 packed rows = one ring slot) from the packed weight matrix; no multicast.
__device__ __forceinline__ void tma_load_slot(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                              uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}


// cuTensorMapEncodeTiled is fetched through the runtime so that the library does not link libcuda
// (it must load on hosts without a driver for the symbol/argument checks).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();
// Packed weights as a 2-D uint32 tensor [KT rows][2N words]; one box = 128 words x 8 rows = one ring slot.
int make_weight_map(CUtensorMap* map, const void* B, int64_t n, int64_t kt);
// The same, kept per (address, n, kt): encoded maps are pure functions of those, so a launch does not re-encode.
int cached_weight_map(CUtensorMap* out, const void* B, int64_t n, int64_t kt);

}  // namespace uniql
