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
  // areas used by the decode linear's own cross-GPU epilogues / prologue (see CommView):
  int64_t block_cap, feat_cap;
  size_t reduce_off, reduce_epoch_off;       // [2][world][block_cap][512] words, then block_cap u32
  size_t gather_off, gather_epoch_off;       // [2][16][feat_cap / 2] words, then feat_cap / 64 u32
  size_t total;
};

static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static ArLayout ar_layout(int world, int64_t max_elems) {
  ArLayout L;
  L.staging_bytes = (size_t)2 * world * max_elems * 4;   // 8-byte words {2 halves, epoch}
  L.flags_off = up256(L.staging_bytes);
  L.epoch_off = L.flags_off;
  // max_elems is read as "16 batch rows of the widest activation row": blocks of 64 columns and features follow
  L.block_cap = max_elems / 1024 > 0 ? max_elems / 1024 : 1;
  L.feat_cap = (max_elems / 16) / 64 * 64;
  if (L.feat_cap < 64) L.feat_cap = 64;
  L.reduce_off = up256(L.epoch_off + (size_t)kArMaxCtas * 4);
  L.reduce_epoch_off = L.reduce_off + (size_t)2 * world * L.block_cap * kFuseBlockWords * 8;
  L.gather_off = up256(L.reduce_epoch_off + (size_t)L.block_cap * 4);
  L.gather_epoch_off = L.gather_off + (size_t)2 * 16 * (L.feat_cap / 2) * 8;
  L.total = up256(L.gather_epoch_off + (size_t)(L.feat_cap / 64) * 4);
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

__device__ __forceinline__ uint4 ld_word2(const uint2* p) {   // two adjacent {data, epoch} words
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
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
    // the first look at the words of four ranks goes out together (two 16-byte loads per rank: one round trip instead
    // of sixteen); a word that has not arrived yet is then polled on its own
    const uint2* slot0 = reinterpret_cast<const uint2*>(mine) + (size_t)parity * p.world * words_per_slot + w0;
    for (int rb = 0; rb < p.world; rb += 4) {
      uint4 wa[4], wb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (rb + j < p.world) {
          wa[j] = ld_word2(slot0 + (size_t)(rb + j) * words_per_slot);
          wb[j] = ld_word2(slot0 + (size_t)(rb + j) * words_per_slot + 2);
        }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (rb + j < p.world) {
          const uint2* slot = slot0 + (size_t)(rb + j) * words_per_slot;
          const uint32_t d0[4] = {wa[j].x, wa[j].z, wb[j].x, wb[j].z};
          const uint32_t e0w[4] = {wa[j].y, wa[j].w, wb[j].y, wb[j].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint2 w = make_uint2(d0[i], e0w[i]);
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
int comm_view(void* comm, CommView* out) {
  uniql_comm* c = (uniql_comm*)comm;
  if (!c || !out) return UNIQL_EINVAL;
  for (int r = 0; r < 8; ++r) out->bufs[r] = c->bufs[r];
  for (int r = 0; r < c->world; ++r)
    if (!c->bufs[r]) return UNIQL_EINVAL;            // uniql_comm_connect has not run
  out->rank = c->rank; out->world = c->world;
  out->reduce = out->gather_out = out->gather_in = 0;
  out->reduce_off = c->layout.reduce_off;
  out->reduce_epoch_off = c->layout.reduce_epoch_off;
  out->block_cap = c->layout.block_cap;
  out->gather_off = c->layout.gather_off;
  out->gather_epoch_off = c->layout.gather_epoch_off;
  out->feat_cap = c->layout.feat_cap;
  out->col_offset = 0;
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
