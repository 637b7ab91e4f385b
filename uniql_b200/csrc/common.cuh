// Shared device helpers and host-side error plumbing for the uniql_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/uniql_b200.h"

namespace uniql {

// ---------------------------------------------------------------- host side
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return UNIQL_ECUDA;
}

#define UNIQL_CUDA_TRY(expr)                         \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) return ::uniql::cuda_fail(_e); \
  } while (0)

// Launch check that does not swallow a sticky error from earlier work.
inline int launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return cuda_fail(e);
  }
  return UNIQL_OK;
}

struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
};
// Cached per device; queried on first use with that device current.
const DeviceInfo& device_info();

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- device side
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  // (a & b) | c in one LOP3
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// Streaming 16-byte load: read-only path, no L1 allocation, L2 evict-first policy.
__device__ __forceinline__ uint4 ld_stream16(const void* p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}

__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint64_t make_evict_last_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint4 ld_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Exact int4 -> fp16 pair conversion used by both the linear and the embedding path.
// Input: a 32-bit word whose bits [3:0] and [19:16] hold two nibbles.  Output: half2 (q_lo - 8, q_hi - 8).
__device__ __forceinline__ uint32_t nib_pair_to_half2_m8(uint32_t w) {
  uint32_t t = lop3_and_or(w, 0x000f000fu, 0x64006400u);       // 1024 + q, exact in fp16
  const uint32_t sub = 0x64086408u;                             // 1032
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<const __half2*>(&sub));
  return *reinterpret_cast<uint32_t*>(&r);
}
// Same for nibbles at bits [7:4] and [23:20]: (1024 + 16 q) / 16 - 72 = q - 8, exact.
__device__ __forceinline__ uint32_t nib_pair_hi_to_half2_m8(uint32_t w) {
  uint32_t t = lop3_and_or(w, 0x00f000f0u, 0x64006400u);
  const uint32_t mul = 0x2c002c00u;                             // 1/16
  const uint32_t add = 0xd480d480u;                             // -72
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<const __half2*>(&mul),
                      *reinterpret_cast<const __half2*>(&add));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  // not volatile: the accumulator operands carry every dependency the scheduler needs
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same MMA, writing fresh accumulators that start from (c0, c1) in both row halves instead of accumulating in place.
__device__ __forceinline__ void mma_m16n8k16_init(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                                  float c0, float c1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}

// Programmatic dependent launch: wait for the preceding kernel in the stream (no-op without the attribute).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace uniql
