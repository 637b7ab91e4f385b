// 4-bit embedding gather for sm_100a.
//
// Replaces w4a16_embedding_lookup_cuda (csrc/embedding/quant_embedding_kernel.cuh:80-114 in UniQL).
// Layout kept from the reference: table int32 [vocab, dim/8]; word w of a row covers elements
// 8w..8w+7 and output element o comes from nibble [0,4,1,5,2,6,3,7][o]; one fp16 scale per row.
// Arithmetic kept from the reference (:47-76): exact q-8 in fp16, one __hmul2 by the row scale.
//
// Mapping: one thread per packed word -> a 4-byte coalesced load and a 16-byte coalesced store
// (a warp reads 128 contiguous bytes and writes 512).  HBM-bound: dim/2 + 2*dim bytes per token.
#include "common.cuh"

namespace uniql {

__global__ void __launch_bounds__(256) w4_embedding_kernel(const int64_t* __restrict__ ids,
                                                           const uint32_t* __restrict__ table,
                                                           const __half* __restrict__ scales,
                                                           uint4* __restrict__ out, int64_t vocab,
                                                           int words_per_row, int* status_word) {
  const int64_t tok = blockIdx.y;
  const int64_t id = ids[tok];
  const bool ok = (id >= 0) && (id < vocab);
  if (!ok && threadIdx.x == 0 && blockIdx.x == 0 && status_word != nullptr)
    atomicOr(status_word, UNIQL_STATUS_BAD_TOKEN_ID);

  __half2 s2 = __half2half2(ok ? scales[id] : __float2half(0.f));
  const uint32_t* row = table + (ok ? id : 0) * (int64_t)words_per_row;
  uint4* orow = out + tok * (int64_t)words_per_row;

  for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < words_per_row; w += gridDim.x * blockDim.x) {
    uint32_t q = ok ? __ldg(row + w) : 0x88888888u;
    uint32_t h0 = nib_pair_to_half2_m8(q);         // elements 0,1  (nibbles 0,4)
    uint32_t h1 = nib_pair_to_half2_m8(q >> 4);    // elements 2,3  (nibbles 1,5)
    uint32_t h2 = nib_pair_to_half2_m8(q >> 8);    // elements 4,5  (nibbles 2,6)
    uint32_t h3 = nib_pair_to_half2_m8(q >> 12);   // elements 6,7  (nibbles 3,7)
    __half2 r0 = __hmul2(*reinterpret_cast<__half2*>(&h0), s2);
    __half2 r1 = __hmul2(*reinterpret_cast<__half2*>(&h1), s2);
    __half2 r2 = __hmul2(*reinterpret_cast<__half2*>(&h2), s2);
    __half2 r3 = __hmul2(*reinterpret_cast<__half2*>(&h3), s2);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&r0);
    o.y = *reinterpret_cast<uint32_t*>(&r1);
    o.z = *reinterpret_cast<uint32_t*>(&r2);
    o.w = *reinterpret_cast<uint32_t*>(&r3);
    orow[w] = o;
  }
}

}  // namespace uniql

extern "C" int uniql_w4_embedding(const int64_t* ids, int64_t n_ids, const void* W, const void* scales,
                                  void* out, int64_t vocab, int64_t dim, int* status_word, void* stream) {
  using namespace uniql;
  if (n_ids < 0 || vocab <= 0 || dim <= 0) return UNIQL_EINVAL;
  if (dim % 8 != 0) return UNIQL_ESHAPE;
  if (n_ids == 0) return UNIQL_OK;
  if (!ids || !W || !scales || !out) return UNIQL_EINVAL;
  if (!aligned16(out) || (reinterpret_cast<uintptr_t>(W) & 3u)) return UNIQL_EINVAL;
  const int words = (int)(dim / 8);
  const int threads = 256;
  int bx = (words + threads - 1) / threads;
  if (bx > 64) bx = 64;
  // gridDim.y is limited to 65535: walk the ids in slabs.
  for (int64_t t0 = 0; t0 < n_ids; t0 += 65535) {
    int64_t nt = n_ids - t0 < 65535 ? n_ids - t0 : 65535;
    dim3 grid(bx, (unsigned)nt);
    w4_embedding_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(
        ids + t0, (const uint32_t*)W, (const __half*)scales, (uint4*)out + t0 * words, vocab, words, status_word);
    int st = launch_status();
    if (st != UNIQL_OK) return st;
  }
  return UNIQL_OK;
}
