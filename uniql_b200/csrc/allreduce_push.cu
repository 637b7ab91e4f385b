// One-shot "push" all-reduce for decode-size messages over NVLink peer memory (sm_100a, one rank per GPU).
//
// The reference has no distributed layer; tensor parallelism of the row-parallel linears (o/down/out_proj)
// needs a sum of [m, hidden] fp16 partials after every such layer.  At decode sizes (8 KB .. 1 MB) the cost of
// a library all-reduce is latency, not bandwidth, so each rank instead *stores* its partial into a slot of every
// peer's staging buffer, raises a flag there, waits (bounded) for the flags of all ranks in its own buffer and
// sums the slots locally in rank order (identical result on every rank).  Data lands in the consumer's own
// memory before it is read; no load ever crosses NVLink and no TMA/multicast is involved.
//
// Memory per rank (allocated once by uniql_comm_create, exported through CUDA IPC):
//   staging[2][world][max_elems/2] x 8 B  every 8-byte word carries two fp16 values and the epoch that wrote it, so
//                                        data and "ready" flag arrive in one atomic store and no fence is needed;
//                                        two parities, so a fast rank can start the next reduction
//   epoch  [kMaxCtas] u32                per-CTA call counter kept on the device (CUDA-graph replay safe)
// CTA c handles elements [c*kChunk, (c+1)*kChunk) and never talks to other CTAs.
#include "common.cuh"
#include "linear_internal.cuh"

#include <stdio.h>

namespace uniql {

constexpr int kArThreads = 256;
constexpr int kArChunk = kArThreads * 8;     // fp16 elements per CTA (4 KB)
constexpr int kArMaxCtas = 256;              // => messages up to 1 MB
constexpr int kArMaxWorld = 8;
constexpr int kArSpinLimit = 1 << 22;

struct ArLayout {
  size_t staging_bytes;   // 2 parities * world slots * max_elems/2 words * 8 bytes
  size_t flags_off, epoch_off;
  size_t fused_staging_off, fused_epoch_off;   // same again for the all-reduce fused into the decode linear
  size_t total;
};

static ArLayout ar_layout(int world, int64_t max_elems) {
  ArLayout L;
  L.staging_bytes = (size_t)2 * world * max_elems * 4;   // 8-byte words {2 halves, epoch}
  L.flags_off = (L.staging_bytes + 255) / 256 * 256;
  L.epoch_off = L.flags_off;
  L.fused_staging_off = (L.epoch_off + (size_t)kArMaxCtas * 4 + 255) / 256 * 256;
  L.fused_epoch_off = L.fused_staging_off + L.staging_bytes;
  L.total = L.fused_epoch_off + (size_t)4096 * 4;      // one epoch counter per column group of the fused linear
  return L;
}

struct ArParams {
  const __half* in;
  __half* out;
  int64_t count, max_elems;
  int rank, world;
  unsigned char* bufs[kArMaxWorld];   // every rank's block, addressable from this GPU
  size_t flags_off, epoch_off;
  int* status_word;
};

__device__ __forceinline__ void st_word(uint2* p, uint32_t data, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_push_kernel(const ArParams p) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  const int cta = blockIdx.x, tid = threadIdx.x;
  unsigned char* mine = p.bufs[p.rank];
  uint32_t* epoch_ctr = reinterpret_cast<uint32_t*>(mine + p.epoch_off) + cta;
  if (tid == 0) { s_epoch = *epoch_ctr + 1; s_fail = 0; }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const uint32_t parity = epoch & 1u;
  const int64_t e0 = (int64_t)cta * kArChunk + tid * 8;
  const bool has = e0 < p.count;           // count is a multiple of 8
  const size_t words_per_slot = (size_t)p.max_elems / 2;
  const size_t w0 = (size_t)e0 / 2;        // first of this thread's four 8-byte words

  // ---- push: four {2 halves, epoch} words into slot `rank` of every rank's staging buffer ----
  if (has) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.in + e0);
    const uint32_t d[4] = {v.x, v.y, v.z, v.w};
    for (int r = 0; r < p.world; ++r) {
      uint2* slot = reinterpret_cast<uint2*>(p.bufs[r]) + ((size_t)parity * p.world + p.rank) * words_per_slot + w0;
#pragma unroll
      for (int i = 0; i < 4; ++i) st_word(slot + i, d[i], epoch);
    }
  }
  // ---- gather: poll my own buffer until each word carries this epoch, sum in rank order (fp32) ----
  if (has) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    bool fail = false;
    for (int r = 0; r < p.world; ++r) {
      const uint2* slot = reinterpret_cast<const uint2*>(mine) + ((size_t)parity * p.world + r) * words_per_slot + w0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint2 w = ld_word(slot + i);
        int it = 0;
        while (w.y != epoch && !fail) {
          if (++it > kArSpinLimit) { fail = true; break; }
          w = ld_word(slot + i);
        }
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    if (fail) s_fail = 1;
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(p.out + e0) = o;
  }
  __syncthreads();
  if (tid == 0) {
    *epoch_ctr = epoch;
    if (s_fail && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);
  }
}

}  // namespace uniql

// ------------------------------------------------------------------------------------------------ C ABI
struct uniql_comm {
  int rank, world;
  int64_t max_elems;
  void* local;                                   // cudaMalloc'ed block of this rank
  unsigned char* bufs[uniql::kArMaxWorld];       // local + IPC-opened peer blocks
  uniql::ArLayout layout;
};

extern "C" size_t uniql_comm_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int uniql_comm_create(int rank, int world, int64_t max_elems, void** comm_out, void* handle_out) {
  using namespace uniql;
  if (!comm_out || !handle_out || world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return UNIQL_EINVAL;
  if (max_elems <= 0 || max_elems % 8 != 0 || max_elems > (int64_t)kArMaxCtas * kArChunk) return UNIQL_ESHAPE;
  uniql_comm* c = new uniql_comm();
  c->rank = rank; c->world = world; c->max_elems = max_elems;
  c->layout = ar_layout(world, max_elems);
  for (int i = 0; i < kArMaxWorld; ++i) c->bufs[i] = nullptr;
  cudaError_t e = cudaMalloc(&c->local, c->layout.total);
  if (e != cudaSuccess) { delete c; return cuda_fail(e); }
  e = cudaMemset(c->local, 0, c->layout.total);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle_out, c->local);
  if (e != cudaSuccess) { cudaFree(c->local); delete c; return cuda_fail(e); }
  c->bufs[rank] = (unsigned char*)c->local;
  *comm_out = c;
  return UNIQL_OK;
}

extern "C" int uniql_comm_connect(void* comm, const void* all_handles) {
  using namespace uniql;
  uniql_comm* c = (uniql_comm*)comm;
  if (!c || !all_handles) return UNIQL_EINVAL;
  const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*)all_handles;
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e);
    c->bufs[r] = (unsigned char*)ptr;
  }
  return UNIQL_OK;
}

extern "C" int uniql_comm_destroy(void* comm) {
  uniql_comm* c = (uniql_comm*)comm;
  if (!c) return UNIQL_OK;
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank && c->bufs[r]) cudaIpcCloseMemHandle(c->bufs[r]);
  cudaFree(c->local);
  delete c;
  return UNIQL_OK;
}

namespace uniql {
int comm_fuse_desc(void* comm, int64_t m, int64_t n, ArFuse* out) {
  uniql_comm* c = (uniql_comm*)comm;
  if (!c || !out) return UNIQL_EINVAL;
  if (m * n > c->max_elems || n / 64 > 4096) return UNIQL_ESHAPE;
  for (int r = 0; r < 8; ++r) out->bufs[r] = c->bufs[r];
  for (int r = 0; r < c->world; ++r)
    if (!c->bufs[r]) return UNIQL_EINVAL;            // uniql_comm_connect has not run
  out->rank = c->rank; out->world = c->world;
  out->staging_off = c->layout.fused_staging_off;
  out->epoch_off = c->layout.fused_epoch_off;
  out->words_per_slot = c->max_elems / 2;
  out->enabled = 1;
  return UNIQL_OK;
}
}  // namespace uniql

extern "C" int uniql_allreduce_push(void* comm, const void* in, void* out, int64_t count, int* status_word,
                                    void* stream) {
  using namespace uniql;
  uniql_comm* c = (uniql_comm*)comm;
  if (!c || count < 0) return UNIQL_EINVAL;
  if (count == 0) return UNIQL_OK;
  if (!in || !out || !aligned16(in) || !aligned16(out)) return UNIQL_EINVAL;
  if (count % 8 != 0 || count > c->max_elems) return UNIQL_ESHAPE;
  ArParams p;
  p.in = (const __half*)in; p.out = (__half*)out; p.count = count; p.max_elems = c->max_elems;
  p.rank = c->rank; p.world = c->world;
  for (int r = 0; r < kArMaxWorld; ++r) p.bufs[r] = c->bufs[r];
  for (int r = 0; r < c->world; ++r)
    if (!p.bufs[r]) return UNIQL_EINVAL;            // uniql_comm_connect has not run
  p.flags_off = c->layout.flags_off; p.epoch_off = c->layout.epoch_off;
  p.status_word = status_word;
  const int ctas = (int)((count + kArChunk - 1) / kArChunk);
  allreduce_push_kernel<<<ctas, kArThreads, 0, (cudaStream_t)stream>>>(p);
  return launch_status();
}
