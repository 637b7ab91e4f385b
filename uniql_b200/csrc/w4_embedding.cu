// 4-bit embedding gather for sm_100a.
//
// Replaces w4a16_embedding_lookup_cuda (csrc/embedding/quant_embedding_kernel.cuh:80-114 in UniQL).
// Layout kept from the reference: table int32 [vocab, dim/8]; word w of a row covers elements
// 8w..8w+7 and output element o comes from nibble [0,4,1,5,2,6,3,7][o]; one fp16 scale per row.
// Arithmetic kept from the reference (:47-76): exact q-8 in fp16, one __hmul2 by the row scale.
//
// Mapping: the (token, packed word) pairs form one flat index space; a thread takes four of them, one block width
// apart, and issues the four id loads, then the four 4-byte word loads and scale loads, before any arithmetic, so four
// dependent id -> row chains are in flight per thread.  Per instruction a warp reads 128 contiguous bytes of a row
// and writes 512 contiguous bytes of the output.  HBM-bound: dim/2 + 2*dim bytes per token.
#include "common.cuh"

namespace uniql {

constexpr int kEmbThreads = 256, kEmbItems = 4;

template <typename Index>
__global__ void __launch_bounds__(kEmbThreads) w4_embedding_kernel(const int64_t* __restrict__ ids,
                                                                   const uint32_t* __restrict__ table,
                                                                   const __half* __restrict__ scales,
                                                                   uint4* __restrict__ out, int64_t vocab,
                                                                   int words_per_row, Index total, int* status_word) {
  const Index i0 = (Index)blockIdx.x * (kEmbThreads * kEmbItems) + threadIdx.x;
  int64_t id[kEmbItems];
  int w[kEmbItems];
  bool valid[kEmbItems], ok[kEmbItems];
#pragma unroll
  for (int j = 0; j < kEmbItems; ++j) {
    const Index i = i0 + (Index)j * kEmbThreads;
    valid[j] = i < total;
    const Index tok = valid[j] ? i / (Index)words_per_row : 0;
    w[j] = valid[j] ? (int)(i - tok * (Index)words_per_row) : 0;
    id[j] = valid[j] ? ids[tok] : 0;
  }
  uint32_t q[kEmbItems];
  __half sc[kEmbItems];
#pragma unroll
  for (int j = 0; j < kEmbItems; ++j) {
    ok[j] = valid[j] && id[j] >= 0 && id[j] < vocab;
    q[j] = ok[j] ? __ldg(table + id[j] * (int64_t)words_per_row + w[j]) : 0x88888888u;   // (8 - 8) * 0: a zero row
    sc[j] = ok[j] ? scales[id[j]] : __float2half(0.f);
  }
#pragma unroll
  for (int j = 0; j < kEmbItems; ++j) {
    if (!valid[j]) continue;
    if (!ok[j] && w[j] == 0 && status_word != nullptr) atomicOr(status_word, UNIQL_STATUS_BAD_TOKEN_ID);
    const __half2 s2 = __half2half2(sc[j]);
    uint32_t h0 = nib_pair_to_half2_m8(q[j]);         // elements 0,1  (nibbles 0,4)
    uint32_t h1 = nib_pair_to_half2_m8(q[j] >> 4);    // elements 2,3  (nibbles 1,5)
    uint32_t h2 = nib_pair_to_half2_m8(q[j] >> 8);    // elements 4,5  (nibbles 2,6)
    uint32_t h3 = nib_pair_to_half2_m8(q[j] >> 12);   // elements 6,7  (nibbles 3,7)
    __half2 r0 = __hmul2(*reinterpret_cast<__half2*>(&h0), s2);
    __half2 r1 = __hmul2(*reinterpret_cast<__half2*>(&h1), s2);
    __half2 r2 = __hmul2(*reinterpret_cast<__half2*>(&h2), s2);
    __half2 r3 = __hmul2(*reinterpret_cast<__half2*>(&h3), s2);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&r0);
    o.y = *reinterpret_cast<uint32_t*>(&r1);
    o.z = *reinterpret_cast<uint32_t*>(&r2);
    o.w = *reinterpret_cast<uint32_t*>(&r3);
    out[i0 + (Index)j * kEmbThreads] = o;             // out is [n_ids, words] uint4: the flat index itself
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
  const int64_t per_block = (int64_t)kEmbThreads * kEmbItems;
  // at most 2^31 - 1 blocks per launch: walk very long id lists in slabs of whole tokens
  const int64_t max_tokens = (((int64_t)1 << 31) - 1) * per_block / words;
  for (int64_t t0 = 0; t0 < n_ids; t0 += max_tokens) {
    const int64_t nt = n_ids - t0 < max_tokens ? n_ids - t0 : max_tokens;
    const int64_t total = nt * words;
    const unsigned blocks = (unsigned)((total + per_block - 1) / per_block);
    uint4* o = (uint4*)out + t0 * words;
    if (total + per_block < ((int64_t)1 << 32))   // 32-bit index arithmetic (the division per item is much cheaper)
      w4_embedding_kernel<uint32_t><<<blocks, kEmbThreads, 0, (cudaStream_t)stream>>>(
          ids + t0, (const uint32_t*)W, (const __half*)scales, o, vocab, words, (uint32_t)total, status_word);
    else
      w4_embedding_kernel<int64_t><<<blocks, kEmbThreads, 0, (cudaStream_t)stream>>>(
          ids + t0, (const uint32_t*)W, (const __half*)scales, o, vocab, words, total, status_word);
    int st = launch_status();
    if (st != UNIQL_OK) return st;
  }
  return UNIQL_OK;
}
