// Decode-regime W4A16 linear (m <= 16) for sm_100a: the dispatch between the two decode kernels, the entry point that
// needs no caller scratch, and the second of the two kernels -- a persistent, slot-balanced, weight-streaming skinny GEMM.
//
// Both kernels replace the small-batch instantiations of UniQL's Marlin kernel
// (csrc/linear/marlin_gemm_kernel.cuh:176-740, tile table :792-800) while consuming the very same
// packed buffers (quantize/quantize_helpers.py:145-165 weight order, :54-62 scale order), and the separate
// launches the reference's blocks make around it: gate_proj / up_proj / act_fn(gate) * up
// (modeling/llama/llama_qblocks.py:48-51), q/k/v (:104-106), the residual add, and the online Hadamard in front of
// down_proj / out_proj (quantize/quant_hadamard_layers.py:16-18).  launch_decode() sends a launch to the CTA-tiled kernel
// of w4a16_gemv.cu (the default, and the only one that talks to other GPUs) or, with UNIQL_B200_DECODE_ENGINE=slot, to
// the kernel below (single GPU).
//
// How the packed layout is consumed.  Packed row kt (16 k-values) holds, for every 64-column block,
// 512 contiguous bytes; lane i of a warp owns bytes 16i..16i+15 = four words j=0..3.  With g = i/4 and
// c = i%4, word j carries W[k, n] for k = 16kt + {2c, 2c+1, 2c+8, 2c+9} and n = 64blk + 16j + g + {0, 8}.
// That is exactly the A-operand fragment of mma.m16n8k16 when the *weights* are the 16-row operand
// (rows = 16 output columns) and the activations are the 8-column operand (columns = batch rows).
// So one 16-byte load per lane feeds four tensor-core instructions per 8 batch rows with no data
// movement between lanes, and all 16 rows of the MMA do useful work even at m = 1.
//
// Work split of the slot kernel.  The unit of work is a *slot*: one quantisation group (128 k-values = 8 packed rows) of
// one 64-column block = 4 KB of packed weights.  A launch is one CTA of 8..16 warps per SM; the T slots of all
// projections of the launch are laid out in one fixed order and warp w of the W = SMs x warps takes slots
// [T w / W, T (w+1) / W): every SM streams the same number of bytes (to within one slot) whatever the matrix shape.
// Each warp owns a ring of two or three slots; one elected lane fills a slot with one 2-D TMA tile (weights, landing on
// the slot's mbarrier: bounded wait, status bit on give-up) while all lanes fetch the group's 64 scales and the
// m x 128 activations with 16-byte asynchronous copies (one commit group per slot).
// A run of slots of one block ends in a 64 x m fp32 tile.  Tiles of a block that spans warps meet in scratch as 8-byte
// words {two values, tag}: the word is its own ready flag, and the warp that holds the block's last slot adds the tiles
// of the lower-numbered warps in a fixed order (bounded polls; no floating-point atomics: same bits on every run),
// clears them, and applies the epilogue: bias, SwiGLU product of a gate/up pair, residual add, fp16 store.  For up to
// four rows the online Hadamard transform of the activations runs in the kernel's own prologue.
//
// Every launch carries the programmatic-dependent-launch attribute, fills its rings, releases its own dependents and only
// then waits for its predecessor.  Measured against the tiled kernel this kernel is slower (its reduction crosses global
// memory); it is kept as a tested alternative.
//
// Roofline: HBM.  Algorithmic bytes per launch = sum over projections of k*n/2 + (k/128)*n*2 + m*n_out*2, + m*k*2.
#include "common.cuh"
#include "linear_internal.cuh"
#include "tma.cuh"

#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

namespace uniql {

constexpr int kSlotScaleBytes = 128;   // 64 fp16 scales
constexpr int kXRowBytes = 272;        // one batch row of one group: 256 bytes + 16 (rows fall on distinct banks)
constexpr int kMaxSeg = 3;             // Hadamard segments a CTA may need in the fused prologue
constexpr int kSegRowBytes = 2048;     // room per (segment, batch row) in the prologue: 512 floats
constexpr int kSegRowStride = 1040;    // bytes between batch rows of a transformed segment (1024 + 16)
constexpr int kMaxPrefetch = 4;
constexpr int kSpinLimit = 1 << 22;    // polls of a tagged word another warp has to write before giving up

// ------------------------------------------------------------------------------------------------ index arithmetic
// Every divisor of the slot arithmetic is a constant of the launch, so divisions are multiplications by a reciprocal
// prepared on the host (an emulated 64-bit division costs ~100 instructions, and a warp does several of them on its
// critical path: range, first slot, tile index).  q = (((n - t) >> 1) + t) >> shift with t = mulhi(magic, n) is exact
// for every 64-bit n (Granlund-Montgomery, round-up variant); powers of two have magic = 0.
struct FastDiv {
  unsigned long long magic;
  int shift;       // -1: divisor 1
  int pad;
};
__host__ __device__ inline unsigned long long mulhi_u64(unsigned long long a, unsigned long long b) {
#ifdef __CUDA_ARCH__
  return __umul64hi(a, b);
#else
  return (unsigned long long)(((unsigned __int128)a * b) >> 64);
#endif
}
__host__ __device__ inline unsigned long long fdiv(unsigned long long n, const FastDiv& d) {
  if (d.shift < 0) return n;
  const unsigned long long t = mulhi_u64(d.magic, n);
  return (((n - t) >> 1) + t) >> d.shift;
}
static FastDiv make_fastdiv(unsigned long long d) {
  FastDiv f{0, -1, 0};
  if (d <= 1) return f;
  int l = 63;
  while (!((d >> l) & 1ull)) --l;                       // floor(log2 d)
  if ((d & (d - 1)) == 0) { f.magic = 0; f.shift = l - 1; return f; }
  const unsigned __int128 num = (unsigned __int128)(1ull << l) << 64;
  unsigned long long m = (unsigned long long)(num / d);
  const unsigned long long rem = (unsigned long long)(num % d);
  m += m;
  const unsigned long long twice = rem + rem;
  if (twice >= d || twice < rem) m += 1;
  f.magic = m + 1;
  f.shift = l;
  return f;
}

// Constants of the slot order, shared by the kernel, the host plan and the host replay.
struct SlotGeom {
  long long T;                    // slots of the launch
  int W, vbT, NG, kc, koff, nchunks, Pc;
  FastDiv dT, dW, dNG, dvbT, dkc;
};

// Slots are ordered chunk by chunk, inside a chunk block by block, inside a block by group.  Without a Hadamard
// prologue there is one chunk (kc = NG): block-major order, the warps that share a block are neighbours.  With it a
// chunk is one Hadamard segment, so that a CTA's slots touch at most kMaxSeg segments of the transformed row.
struct SlotIt {
  int c, vb, g, g_lo, g_hi;
};
__host__ __device__ inline int chunk_lo(int c, int kc, int koff) { const int v = c * kc - koff; return v < 0 ? 0 : v; }
__host__ __device__ inline int chunk_hi(int c, int kc, int koff, int NG) {
  const int v = (c + 1) * kc - koff;
  return v > NG ? NG : v;
}
// first slot of warp w
__host__ __device__ inline long long warp_begin(const SlotGeom& G, int w) { return (long long)fdiv((unsigned long long)G.T * w, G.dW); }
__host__ __device__ inline SlotIt slot_decode(const SlotGeom& G, long long s) {
  SlotIt it;
  const int q = (int)fdiv((unsigned long long)s, G.dvbT);
  it.c = (int)fdiv((unsigned long long)(q + G.koff), G.dkc);
  it.g_lo = chunk_lo(it.c, G.kc, G.koff);
  it.g_hi = chunk_hi(it.c, G.kc, G.koff, G.NG);
  const int w = it.g_hi - it.g_lo;
  const int rem = (int)(s - (long long)G.vbT * it.g_lo);
  it.vb = rem / w;                                      // w <= kc is small and varies at the row's edges: plain division
  it.g = it.g_lo + (rem - it.vb * w);
  return it;
}
// CH = false: a single chunk, so c, g_lo and g_hi are constants and cost no registers
template <bool CH>
__host__ __device__ __forceinline__ SlotIt slot_at(const SlotGeom& G, long long s) {
  if (CH) return slot_decode(G, s);
  SlotIt it;
  it.c = 0; it.g_lo = 0; it.g_hi = G.NG;
  it.vb = (int)fdiv((unsigned long long)s, G.dNG);
  it.g = (int)(s - (long long)it.vb * G.NG);
  return it;
}
template <bool CH>
__host__ __device__ __forceinline__ void slot_next(const SlotGeom& G, SlotIt& it) {
  if (!CH) {
    if (++it.g == G.NG) { it.g = 0; ++it.vb; }
    return;
  }
  if (++it.g == it.g_hi) {
    it.g = it.g_lo;
    if (++it.vb == G.vbT) {
      it.vb = 0;
      ++it.c;
      it.g_lo = it.g_hi;
      it.g_hi = it.g_hi + G.kc > G.NG ? G.NG : it.g_hi + G.kc;
      it.g = it.g_lo;
    }
  }
}
// warp that owns slot s: the largest w with T w / W <= s
__host__ __device__ inline int warp_of_slot(const SlotGeom& G, long long s) {
  return (int)fdiv((unsigned long long)(s + 1) * G.W - 1, G.dT);
}
// Number of tiles block vb receives inside chunk [g_lo, g_hi): the warps whose slot ranges touch it.  With fewer slots
// than warps every busy warp holds exactly one slot (and idle warps sit between them), so each slot is its own tile.
__host__ __device__ inline int runs_of(const SlotGeom& G, int vb, int g_lo, int g_hi) {
  const int w = g_hi - g_lo;
  if (G.T < G.W) return w;
  const long long first = (long long)G.vbT * g_lo + (long long)vb * w;
  return warp_of_slot(G, first + w - 1) - warp_of_slot(G, first) + 1;
}
// Index of a run among the tiles of its block and chunk: `first` is the first slot of the block inside the chunk,
// `run_first` the first slot of the run, wg the warp that holds it.
__host__ __device__ inline int run_index(const SlotGeom& G, long long first, long long run_first, int wg) {
  if (G.T < G.W) return (int)(run_first - first);
  return wg - warp_of_slot(G, first);
}

struct DecodeProj {
  const __half* S;
  const __half* bias;
  __half* D;
  long long ldd;
  int N, n_out;
};

struct DecodeParams {
  CUtensorMap wmap[kMaxProj];
  DecodeProj proj[kMaxProj];
  int vb_start[kMaxProj + 1];     // first virtual block of each projection (plain order)
  const __half* A;
  long long lda;
  const __half* residual;
  long long ldr;
  uint2* partials;                // partial tiles as tagged words {fp32 bits, tag}: [block][chunk][Pc][M][64]
  uint32_t tag;                   // tag of this launch's words (never 0: consumed words are cleared to 0)
  int* status_word;
  SlotGeom G;                     // T slots over W warps; k cut into chunks of kc groups (chunk c = local groups
                                  // [c kc - koff, (c+1) kc - koff)); Pc tiles reserved per block and chunk
  int M, nproj, epilogue;
  int xbytes;                     // bytes of staged activations per ring slot
  int had;                        // 1: the activations are H a / sqrt(dim), formed by each CTA for the chunks it streams
  int hP, hlogP, hlogQ, hMdim;    // dim = base * Q * P, P <= 512 the segment length, Mdim = base * Q segments
  int seg0;                       // global segment index of chunk 0
  float hscale;
  unsigned long long hsign[40];   // base matrix: bit a' of hsign[a] set <=> H[a][a'] = -1
  const unsigned char* pf_ptr[kMaxPrefetch];   // byte ranges to pull into L2 when this launch's own stream ends
  long long pf_lines[kMaxPrefetch];            // (the weights of the launches that follow), in 128-byte lines
  int npf;
};

// ------------------------------------------------------------------------------------------------ device helpers
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol)
      : "memory");
}
// Per-thread 16-byte asynchronous copy global -> shared (no copy-engine request, no registers held).  The copies of one
// ring slot form one commit group; a slot is consumed after cp.async.wait_group has retired its group.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Predicated forms: one instruction under a predicate instead of a divergent branch around it (the source address is
// not touched when the predicate is false).
__device__ __forceinline__ void cp_async16_if(bool pred, uint32_t dst, const void* src) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %0, 0;\n\t@p cp.async.cg.shared.global [%1], [%2], 16;\n\t}"
      ::"r"((int)pred), "r"(dst), "l"(src)
      : "memory");
}
// Lane `pred` arms the slot's barrier with the tile's byte count and issues the 2-D TMA tile (no multicast).
__device__ __forceinline__ void tma_slot_if(bool pred, uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                            uint64_t pol) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %0, 0;\n\t"
      "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%5], 4096;\n\t"
      "@p cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%1], [%2, {%3, %4}], [%5], %6;\n\t}"
      ::"r"((int)pred), "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// A partial sum travels between warps as an 8-byte word {fp32 bits, tag}: one store, one load, and the tag says whether
// the value of THIS launch has arrived -- no fence and no counter between producer and consumer.
template <int BYTE_OFF>
__device__ __forceinline__ void st_tagged(uint2* p, float v, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0 + %3], {%1, %2};"
               ::"l"(p), "r"(__float_as_uint(v)), "r"(tag), "n"(BYTE_OFF)
               : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2(const uint2* p) {   // two adjacent words
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void clear_tagged2(uint2* p) {
  asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1, %1, %1, %1};" ::"l"(p), "r"(0u) : "memory");
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ void proj_of_block(const DecodeParams& p, int vb, int& pi, int& lb) {
  if (p.epilogue == UNIQL_EPILOGUE_SWIGLU) {
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

// One quantisation group of one 64-column block out of a ring slot.  Nibbles become fp16 values (1024 + q) and
// (64 + q) by a single LOP3 each; the offsets come out again through `corr`, the product of the same activations
// with the constant weights (1032 | 72):  sum (off + q) x - sum (off + 8) x = sum (q - 8) x.
template <int MT>
__device__ __forceinline__ void decode_group(uint32_t wslot, uint32_t xl, uint32_t xts, float (&accg)[MT][4][4],
                                             float (&corr)[MT][4], uint32_t kc_lo, uint32_t kc_hi) {
  const uint32_t kcorr[4] = {kc_lo, kc_lo, kc_hi, kc_hi};   // halves 1032, 1032, 72, 72
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint4 w4 = lds128(wslot + u * 512);
    uint32_t b0[MT], b1[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      b0[t] = lds32(xl + t * xts + u * 32);
      b1[t] = lds32(xl + t * xts + u * 32 + 16);
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      if (u == 0) mma_m16n8k16_init(corr[t], kcorr, b0[t], b1[t], 0.f, 0.f);
      else mma_m16n8k16(corr[t], kcorr, b0[t], b1[t]);
    }
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
        if (u == 0) mma_m16n8k16_init(accg[t][j], a, b0[t], b1[t], 0.f, 0.f);
        else mma_m16n8k16(accg[t][j], a, b0[t], b1[t]);
      }
    }
  }
}

// Stores a warp's accumulators as tagged words and clears them.  `lane_tile` points at (row 2c, column g) of the tile.
template <int MT, int T = 0, int J = 0, int R = 0>
__device__ __forceinline__ void flush_tile(uint2* lane_tile, float (&acc)[MT][4][4], int row0, int M, uint32_t tag) {
  if constexpr (T < MT) {
    constexpr int kOff = ((8 * T + (R & 1)) * 64 + 16 * J + 8 * (R >> 1)) * 8;
    if (row0 + 8 * T + (R & 1) < M) st_tagged<kOff>(lane_tile, acc[T][J][R], tag);
    acc[T][J][R] = 0.f;
    if constexpr (R < 3) flush_tile<MT, T, J, R + 1>(lane_tile, acc, row0, M, tag);
    else if constexpr (J < 3) flush_tile<MT, T, J + 1, 0>(lane_tile, acc, row0, M, tag);
    else flush_tile<MT, T + 1, 0, 0>(lane_tile, acc, row0, M, tag);
  }
}

// Final values of two adjacent columns of one batch row -> fp16 (bias, optional SwiGLU partner, optional residual),
// stored to D.
__device__ __forceinline__ void store_pair(const DecodeParams& p, const DecodeProj& pr, const DecodeProj& pr2, int m,
                                           int n0, float2 v, float2 v2, bool swiglu) {
  if (n0 >= pr.n_out) return;
  const bool two = n0 + 1 < pr.n_out;
  if (pr.bias) {
    v.x += __half2float(pr.bias[n0]);
    if (two) v.y += __half2float(pr.bias[n0 + 1]);
  }
  __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y);
  if (swiglu) {
    // act_fn(gate) * up with the roundings of the separate modules: fp16 gate, fp16 up, fp16 SiLU, fp16 product
    if (pr2.bias) {
      v2.x += __half2float(pr2.bias[n0]);
      if (two) v2.y += __half2float(pr2.bias[n0 + 1]);
    }
    const __half u0 = __float2half_rn(v2.x), u1 = __float2half_rn(v2.y);
    const __half a0 = __float2half_rn(silu_f(__half2float(h0))), a1 = __float2half_rn(silu_f(__half2float(h1)));
    h0 = __float2half_rn(__half2float(a0) * __half2float(u0));
    h1 = __float2half_rn(__half2float(a1) * __half2float(u1));
  }
  if (p.residual) {
    const __half* r = p.residual + (size_t)m * p.ldr + n0;
    h0 = __float2half_rn(__half2float(h0) + __half2float(r[0]));
    if (two) h1 = __float2half_rn(__half2float(h1) + __half2float(r[1]));
  }
  __half* d = pr.D + (size_t)m * pr.ldd + n0;
  if (two && ((reinterpret_cast<uintptr_t>(d) & 3u) == 0)) {
    *reinterpret_cast<__half2*>(d) = __halves2half2(h0, h1);
  } else {
    d[0] = h0;
    if (two) d[1] = h1;
  }
}

// Finishes one block (or one gate/up pair of blocks): the calling warp -- the one that streamed the block's last slot --
// waits for the tiles of all the warps that worked on it (words tagged with this launch's tag, bounded poll), adds
// them up in a fixed order and finishes the 64 columns, two per lane.  Consumed words are cleared to tag 0 for the
// launches to come.  Returns false if the wait gave up.
__device__ __forceinline__ bool finish_block(const DecodeParams& p, int unit, int lane) {
  const bool swiglu = p.epilogue == UNIQL_EPILOGUE_SWIGLU;
  const size_t tile_elems = (size_t)p.M * 64;   // words per tile
  bool ok = true;
  int pi, lb;
  proj_of_block(p, swiglu ? 2 * unit : unit, pi, lb);
  const DecodeProj& pr = p.proj[pi];
  const DecodeProj& pr2 = p.proj[swiglu ? 1 : pi];
  // tiles per chunk of the block(s), chunk cc in lane cc % 32
  int pc[2][3];
#pragma unroll
  for (int wh = 0; wh < 2; ++wh)
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int cc = lane + 32 * q;
      pc[wh][q] = 0;
      if ((wh == 0 || swiglu) && cc < p.G.nchunks)
        pc[wh][q] = runs_of(p.G, swiglu ? 2 * unit + wh : unit, chunk_lo(cc, p.G.kc, p.G.koff),
                            chunk_hi(cc, p.G.kc, p.G.koff, p.G.NG));
    }
  const int total = p.G.nchunks * p.G.Pc;
  for (int m = 0; m < p.M; ++m) {
    float2 v[2];
#pragma unroll
    for (int wh = 0; wh < 2; ++wh) {
      v[wh] = make_float2(0.f, 0.f);
      if (wh == 1 && !swiglu) continue;
      const int vb = swiglu ? 2 * unit + wh : unit;
      uint2* base = p.partials + (size_t)vb * p.G.nchunks * p.G.Pc * tile_elems + (size_t)m * 64 + 2 * lane;
      // tiles in (chunk, run) order, up to 8 independent 16-byte loads in flight, summed in that order; (cc, jj) walk
      // the reserved places of the block and `runs` says how many of a chunk's places hold a tile
      int cc = 0, jj = 0;
      int runs = __shfl_sync(0xffffffffu, pc[wh][0], 0);
      for (int i0 = 0; i0 < total; i0 += 8) {
        uint4 t8[8];
        uint32_t use = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if ((i0 + q < total) && (jj < runs)) {
            use |= 1u << q;
            t8[q] = ld_tagged2(base + (size_t)(i0 + q) * tile_elems);
          }
          if (++jj == p.G.Pc) {
            jj = 0;
            ++cc;
            const int src = cc < 32 ? pc[wh][0] : cc < 64 ? pc[wh][1] : pc[wh][2];
            runs = __shfl_sync(0xffffffffu, src, cc & 31);
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if ((use >> q) & 1u) {
            uint2* src = base + (size_t)(i0 + q) * tile_elems;
            int spin = 0;
            while ((t8[q].y != p.tag || t8[q].w != p.tag) && ok) {
              if (++spin > kSpinLimit) { ok = false; break; }
              t8[q] = ld_tagged2(src);
            }
            v[wh].x += __uint_as_float(t8[q].x);
            v[wh].y += __uint_as_float(t8[q].z);
            clear_tagged2(src);
          }
      }
    }
    const int n0 = lb * 64 + 2 * lane;
    store_pair(p, pr, pr2, m, n0, v[0], v[1], swiglu);
  }
  return ok;
}

// Hadamard prologue of a CTA: forms, in shared memory, the segments of  H a / sqrt(dim)  that the CTA's slots multiply
// with (nseg consecutive segments from global segment seg0 + c_first, every batch row), rounded to fp16.
// dim = Mdim x P with commuting factors: segment s of the result is the P-point Walsh-Hadamard transform of
// sum_a' sign(s, a') a[a' P .. a' P + P).  Returns false if a wait gave up (none in this version).
__device__ __noinline__ bool hadamard_prologue(const DecodeParams& p, uint8_t* area, uint32_t* s_mask, int c_first,
                                               int nseg, int nthreads) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int P = p.hP, half_p = P >> 1;
  const int Q1 = (1 << p.hlogQ) - 1;
  float* zbuf = reinterpret_cast<float*>(area);
  bool ok = true;
  // sign of the (segment, source segment) pairs: base matrix on the slow index, Sylvester on the fast one
  if (warp < nseg) {
    const int seg = p.seg0 + c_first + warp;
    for (int i = 0; i < 3; ++i) {
      const int ap = lane + 32 * i;
      int neg = 0;
      if (ap < p.hMdim) {
        neg = (int)((p.hsign[seg >> p.hlogQ] >> (ap >> p.hlogQ)) & 1ull);
        neg ^= __popc((unsigned)((seg & Q1) & (ap & Q1))) & 1;
      }
      const uint32_t mk = __ballot_sync(0xffffffffu, neg);
      if (lane == 0) s_mask[warp * 3 + i] = mk;
    }
  }
  __syncthreads();
  // z[seg][row][b] = sum_a' sign(seg, a') a[row][a' P + b]: a thread owns two adjacent b of one row and, when there
  // are threads to spare (one batch row), every `nsplit`-th source segment; the split sums meet in shared memory
  const int nitems = p.M * half_p;
  const int nsplit = (p.M == 1 && 2 * nitems <= nthreads) ? 2 : 1;
  for (int it0 = tid; it0 < nitems * nsplit; it0 += nthreads) {
    const int split = it0 >= nitems ? 1 : 0;
    const int item = it0 - split * nitems;
    const int row = item >> (p.hlogP - 1), cp = item & (half_p - 1);
    float2 z[kMaxSeg];
#pragma unroll
    for (int s = 0; s < kMaxSeg; ++s) z[s] = make_float2(0.f, 0.f);
    constexpr int NB = 16;                   // source segments fetched per round trip
    for (int a0 = split; a0 < p.hMdim; a0 += NB * nsplit) {
      uint32_t hv[NB];
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.A + (size_t)row * p.lda) + cp;
#pragma unroll
      for (int i = 0; i < NB; ++i)
        if (a0 + i * nsplit < p.hMdim) hv[i] = __ldcg(src + (size_t)(a0 + i * nsplit) * half_p);
#pragma unroll
      for (int i = 0; i < NB; ++i)
        if (a0 + i * nsplit < p.hMdim) {
          const int ap = a0 + i * nsplit;
          // flip the sign bits of the two halves where the matrix entry is -1
#pragma unroll
          for (int s = 0; s < kMaxSeg; ++s)
            if (s < nseg) {
              const uint32_t flip = ((s_mask[s * 3 + (ap >> 5)] >> (ap & 31)) & 1u) * 0x80008000u;
              const uint32_t hs = hv[i] ^ flip;
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hs));
              z[s].x += f.x;
              z[s].y += f.y;
            }
        }
    }
#pragma unroll
    for (int s = 0; s < kMaxSeg; ++s)
      if (s < nseg) *reinterpret_cast<float2*>(zbuf + (size_t)((split * kMaxSeg + s) * p.M + row) * 512 + 2 * cp) = z[s];
  }
  __syncthreads();
  if (nsplit == 2) {
    for (int i = tid; i < nseg * half_p; i += nthreads) {      // one batch row here: (segment, column pair)
      const int sgi = i >> (p.hlogP - 1), cp = i & (half_p - 1);
      float2* d = reinterpret_cast<float2*>(zbuf + (size_t)sgi * 512 + 2 * cp);
      const float2 e = *reinterpret_cast<const float2*>(zbuf + (size_t)(kMaxSeg + sgi) * 512 + 2 * cp);
      d->x += e.x;
      d->y += e.y;
    }
    __syncthreads();
  }
  // P-point Walsh-Hadamard transform of every (segment, row) vector, radix 8 / 4 / 2 out of shared memory
  const int ntask = nseg * p.M;
  for (int h = 1; h < P;) {
    const int rem = P / h;
    const int R = rem >= 8 ? 8 : rem;
    const int lh = __ffs(h) - 1, lgr = p.hlogP - (R == 8 ? 3 : R == 4 ? 2 : 1);   // log2(groups per vector)
    for (int idx = tid; idx < (ntask << lgr); idx += nthreads) {
      const int task = idx >> lgr, gi = idx & ((1 << lgr) - 1);
      const int low = gi & (h - 1), high = gi >> lh;
      float* q = zbuf + (size_t)task * 512 + (size_t)high * h * R + low;
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < R) v[i] = q[(size_t)i * h];
#pragma unroll
      for (int st = 1; st < 8; st <<= 1)
        if (st < R) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i < R && !(i & st)) {
              const float a = v[i], b = v[i | st];
              v[i] = a + b;
              v[i | st] = a - b;
            }
        }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < R) q[(size_t)i * h] = v[i];
    }
    __syncthreads();
    h *= R;
  }
  // scale, round to fp16 (as the separate Hadamard module would), repack as rows of kSegRowStride bytes
  uint32_t packed[12];
  const int npack = ntask * half_p;
#pragma unroll
  for (int i = 0; i < 12; ++i) {
    const int item = tid + i * nthreads;
    if (item < npack) {
      const int task = item >> (p.hlogP - 1), cp = item & (half_p - 1);
      const float2 f = *reinterpret_cast<const float2*>(zbuf + (size_t)task * 512 + 2 * cp);
      const __half2 hh = __floats2half2_rn(f.x * p.hscale, f.y * p.hscale);
      packed[i] = *reinterpret_cast<const uint32_t*>(&hh);
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 12; ++i) {
    const int item = tid + i * nthreads;
    if (item < npack) {
      const int task = item >> (p.hlogP - 1), cp = item & (half_p - 1);
      *reinterpret_cast<uint32_t*>(area + (size_t)task * kSegRowStride + cp * 4) = packed[i];
    }
  }
  __syncthreads();
  return ok;
}

#ifdef UNIQL_DECODE_TIMING
// Development aid (never defined in the shipped build): per-warp timestamps of the phases of one launch.
__device__ unsigned long long g_decode_stamps[8][4096];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(k) do { if (lane == 0 && wg < 4096) g_decode_stamps[k][wg] = gtime(); } while (0)
#else
#define STAMP(k) do { } while (0)
#endif

template <int MT, int WARPS, int MINB, bool HAD, int kRing>
__global__ void __launch_bounds__(WARPS * 32, MINB) w4a16_decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_bars[WARPS * kRing];
  __shared__ uint32_t s_mask[kMaxSeg][3];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int wg = blockIdx.x * WARPS + warp;
  STAMP(0);
  const long long s0 = warp_begin(p.G, wg), s1 = warp_begin(p.G, wg + 1);
  const int nsl = (int)(s1 - s0);

  // ---- shared memory: [weights: WARPS x kRing x 4 KB][scales: WARPS x kRing x 128 B][activations] ----
  const uint32_t smem_base = smem_addr(smem_raw);
  const uint32_t wring = smem_base + warp * (kRing * kSlotBytes);
  const uint32_t sring = smem_base + WARPS * (kRing * kSlotBytes) + warp * (kRing * kSlotScaleBytes);
  const uint32_t xarea = smem_base + WARPS * (kRing * (kSlotBytes + kSlotScaleBytes));
  const uint32_t xring = xarea + warp * (kRing * p.xbytes);
  const uint32_t bar0 = smem_addr(&s_bars[warp * kRing]);
  const uint64_t pol_w = make_evict_first_policy();

  if (lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&p.wmap[0]) : "memory");
    // the barrier of a slot tracks its weight tile (one arrival with the byte count, by the issuing lane); the lanes'
    // asynchronous copies of the group's scales and activations are tracked by commit groups
    for (int s = 0; s < kRing; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  // One copy-engine request per slot (the 4 KB weight tile); the 64 scales of the group and the m x 128 activations
  // travel as per-thread 16-byte asynchronous copies: small bulk copies cost the copy engine as much as a tile.
  // The issue side keeps its operands as running values: inside a run of slots of one block only the group advances.
  SlotIt it_issue = slot_at<HAD>(p.G, s0);
  const CUtensorMap* is_map = &p.wmap[0];
  int is_x = 0;                              // word coordinate of the block in the packed row
  const __half* is_sp = p.proj[0].S;         // this lane's 8 scales of the slot to issue (lanes 0..7)
  long long is_sn = 0;                       // halves between consecutive scale rows
  auto issue_block = [&]() {                 // operands of the block it_issue points at
    int pi, lb;
    proj_of_block(p, it_issue.vb, pi, lb);
    is_map = &p.wmap[pi];
    is_x = lb * 128;
    is_sn = p.proj[pi].N;
    is_sp = p.proj[pi].S + ((size_t)it_issue.g * is_sn + (size_t)lb * 64 + (lane & 7) * 8);
  };
  // activations: lane l copies chunk l % 16 of batch row l / 16 (+ 2 rows per further pass)
  const __half* xsrc0 = p.A + (size_t)(lane >> 4) * p.lda + (lane & 15) * 8;
  const uint32_t xdst0 = xring + (lane >> 4) * kXRowBytes + (lane & 15) * 16;
  auto issue_weights = [&](int slot) {       // all lanes
    const uint32_t bar = bar0 + slot * 8;
    tma_slot_if(lane == 0, wring + slot * kSlotBytes, is_map, is_x, 8 * it_issue.g, bar, pol_w);
    cp_async16_if(lane < 8, sring + slot * kSlotScaleBytes + lane * 16, is_sp);
  };
  auto issue_acts = [&](int slot, int grp) {  // all lanes: 16 chunks of 16 bytes per batch row
    const __half* src = xsrc0 + (size_t)grp * 128;
    const uint32_t dst = xdst0 + slot * p.xbytes;
    cp_async16_if(lane < 16 * p.M, dst, src);
    for (int r2 = 2; r2 < p.M; r2 += 2)
      cp_async16_if(lane + 16 * r2 < 16 * p.M, dst + r2 * kXRowBytes, src + (size_t)r2 * p.lda);
  };
  auto issue_next = [&]() {                  // advance the issue side by one slot
    const int vb_before = it_issue.vb;
    slot_next<HAD>(p.G, it_issue);
    if (it_issue.vb != vb_before) {
      if (it_issue.vb < p.G.vbT) issue_block();
    } else {
      is_sp += is_sn;
    }
  };

  // When this warp's own stream ends it asks L2 for its share of the weights the following launches will stream:
  // HBM then stays busy while this launch drains and the next one starts, and the next one finds its first
  // megabytes in L2.  Plain per-line prefetches (hints: they cost no registers and never fault).
  auto issue_prefetch = [&]() {
    const long long nthreads_all = (long long)gridDim.x * (WARPS * 32);
    const long long gtid = (long long)blockIdx.x * (WARPS * 32) + tid;
    for (int r = 0; r < p.npf; ++r)
      for (long long l = gtid; l < p.pf_lines[r]; l += nthreads_all)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.pf_ptr[r] + l * 128));
  };

  // ---- start streaming weights before anything else ----
  if (nsl > 0) issue_block();
  int g_pre[kRing];
#pragma unroll
  for (int s = 0; s < kRing; ++s) {
    g_pre[s] = it_issue.g;
    if (s < nsl) {
      issue_weights(s);
      issue_next();
    }
  }
  // Let the next kernel in the stream start its own weight prefetch, then wait for the producer of the activations.
  STAMP(1);
  pdl_launch_dependents();
  pdl_wait();
  STAMP(2);

  bool timed_out = false;
  // chunk range of this CTA (Hadamard prologue) -- CTA-uniform
  int c_first = 0;
  if (HAD) {
    const long long cs0 = warp_begin(p.G, blockIdx.x * WARPS), cs1 = warp_begin(p.G, (blockIdx.x + 1) * WARPS);
    if (cs1 > cs0) {
      c_first = slot_decode(p.G, cs0).c;
      const int c_last = slot_decode(p.G, cs1 - 1).c;
      int nseg = c_last - c_first + 1;
      if (nseg > kMaxSeg) nseg = kMaxSeg;                 // excluded by the host plan
      if (!hadamard_prologue(p, smem_raw + (xarea - smem_base), &s_mask[0][0], c_first, nseg, WARPS * 32)) timed_out = true;
    }
  }
  // one commit group per ring slot, empty ones included: the group of slot i is then always followed by exactly
  // kRing - 1 younger groups when slot i is consumed (the scales fetched above ride in the first group)
#pragma unroll
  for (int s = 0; s < kRing; ++s) {
    if (!HAD && s < nsl) issue_acts(s, g_pre[s]);
    cp_async_commit();
  }

  // this lane's B-fragment origin: batch row g (tile 0) and 8 + g (tile 1), clamped to a row that exists --
  // batch columns past m only feed accumulator columns that are never stored
  const int row_t0 = min(g, p.M - 1), row_t1 = min(8 + g, p.M - 1);
  const uint32_t xrs = HAD ? (uint32_t)kSegRowStride : (uint32_t)kXRowBytes;
  const uint32_t xl_off = (uint32_t)row_t0 * xrs + c * 4;
  const uint32_t xts = (uint32_t)(row_t1 - row_t0) * xrs;

  float acc[MT][4][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[t][j][r] = 0.f;
  // the constant operand of the offset-correction MMA, kept in registers (opaque to the compiler: no re-materialising)
  uint32_t kc_lo, kc_hi;
  asm volatile("mov.b32 %0, 0x64086408;" : "=r"(kc_lo));
  asm volatile("mov.b32 %0, 0x54805480;" : "=r"(kc_hi));

  if (nsl == 0) issue_prefetch();
  SlotIt it = slot_at<HAD>(p.G, s0);
  int run_cnt = 0;
  const size_t tile_elems = (size_t)p.M * 64;
  int slot = 0;
  uint32_t parity = 0;
  int fin_first = 0, fin_cnt = 0;
  for (int i = 0; i < nsl; ++i) {
    cp_async_wait<kRing - 1>();          // this lane's copies for slot i have landed ...
    __syncwarp();                        // ... and so have the other lanes'
    if (!mbar_wait(bar0 + slot * 8, parity)) timed_out = true;
    if (i == 0) STAMP(3);
    if (i == nsl - 1) STAMP(4);
    const uint4 sc = lds128(sring + slot * kSlotScaleBytes + 16 * g);
    uint32_t xl;
    if (HAD)
      xl = xarea + (uint32_t)((it.c - c_first) * p.M) * kSegRowStride + (uint32_t)(it.g + p.G.koff - it.c * p.G.kc) * 256u + xl_off;
    else
      xl = xring + slot * p.xbytes + xl_off;
    float accg[MT][4][4], corr[MT][4];
    decode_group<MT>(wring + slot * kSlotBytes + lane * 16, xl, xts, accg, corr, kc_lo, kc_hi);
    // the slot has been read by every lane: hand it back to the copy engine
    __syncwarp();
    if (i + kRing < nsl) {
      issue_weights(slot);
      if (!HAD) issue_acts(slot, it_issue.g);
      issue_next();
    }
    cp_async_commit();
    if (i == nsl - 1) issue_prefetch();
    // ---- apply this group's scales: lane holds s[64blk + 8g + 2j + b] for j=0..3, b=0..1 ----
    const __half2* sh = reinterpret_cast<const __half2*>(&sc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 sf = __half22float2(sh[j]);   // .x -> columns 16j+g, .y -> 16j+g+8
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        acc[t][j][0] = fmaf(accg[t][j][0] - corr[t][0], sf.x, acc[t][j][0]);
        acc[t][j][1] = fmaf(accg[t][j][1] - corr[t][1], sf.x, acc[t][j][1]);
        acc[t][j][2] = fmaf(accg[t][j][2] - corr[t][2], sf.y, acc[t][j][2]);
        acc[t][j][3] = fmaf(accg[t][j][3] - corr[t][3], sf.y, acc[t][j][3]);
      }
    }
    if (i == nsl - 1) STAMP(5);
    ++run_cnt;
    const bool run_end = (i == nsl - 1) || (it.g + 1 == it.g_hi);
    if (run_end) {
      // ---- this warp's tile of block it.vb goes to scratch as tagged words ----
      const int wc = it.g_hi - it.g_lo;
      const long long first = (long long)p.G.vbT * it.g_lo + (long long)it.vb * wc;
      const int jrun = run_index(p.G, first, s0 + i - (run_cnt - 1), wg);
      // this lane's words: batch rows 8t + 2c + (r & 1), columns 16j + g + 8 (r >> 1): one base, constant offsets
      uint2* tile = p.partials + ((size_t)((size_t)it.vb * p.G.nchunks + it.c) * p.G.Pc + jrun) * tile_elems + (2 * c) * 64 + g;
      const uint32_t tag = p.tag;
      flush_tile<MT>(tile, acc, 2 * c, p.M, tag);
      // The warp that holds the LAST slot of a block (of the up block of a gate/up pair) finishes it: it waits for the
      // tiles of the warps before it -- always warps of lower index, in CTAs that were dispatched no later than its
      // own, so the wait cannot deadlock -- adds them up in a fixed order and applies the epilogue.
      const bool swiglu = p.epilogue == UNIQL_EPILOGUE_SWIGLU;
      const int unit = swiglu ? (it.vb >> 1) : it.vb;
      const bool last = (it.g == p.G.NG - 1) && (!swiglu || (it.vb & 1));
      // Finishing waits for other warps' tiles, so it is put off until this warp has stored all of its own: no warp
      // ever waits while it still owes a tile to somebody else.  The blocks a warp finishes are consecutive.
      if (last) {
        if (fin_cnt == 0) fin_first = unit;
        ++fin_cnt;
      }
      if (i == nsl - 1) STAMP(6);
      run_cnt = 0;
    }
    slot_next<HAD>(p.G, it);
    if (++slot == kRing) { slot = 0; parity ^= 1u; }
  }
  for (int u = 0; u < fin_cnt; ++u)
    if (!finish_block(p, fin_first + u, lane)) timed_out = true;
  STAMP(7);
  if (timed_out && p.status_word) atomicOr(p.status_word, UNIQL_STATUS_WAIT_TIMEOUT);
}

#ifdef UNIQL_DECODE_TIMING
}  // namespace uniql
extern "C" int uniql_debug_read_stamps(unsigned long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, uniql::g_decode_stamps, sizeof(unsigned long long) * 8 * 4096);
}
namespace uniql {
#endif

// ------------------------------------------------------------------------------------------------ host side
static int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

EncodeTiledFn encode_tiled_fn() {
  static const EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return (EncodeTiledFn)ptr;
    return (EncodeTiledFn) nullptr;
  }();
  return fn;
}

int make_weight_map(CUtensorMap* map, const void* B, int64_t n, int64_t kt) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return cuda_fail(cudaErrorNotSupported);
  cuuint64_t dims[2] = {(cuuint64_t)(2 * n), (cuuint64_t)kt};
  cuuint64_t strides[1] = {(cuuint64_t)(2 * n) * 4};
  cuuint32_t box[2] = {128, 8};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(B), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  return UNIQL_OK;
}

// Encoded tensor maps are pure functions of (address, n, k): keep them instead of encoding on every launch.
struct MapKey {
  const void* B;
  int64_t n, kt;
  bool operator==(const MapKey& o) const { return B == o.B && n == o.n && kt == o.kt; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.B) ^ (std::hash<int64_t>()(k.n) * 1000003u) ^ (std::hash<int64_t>()(k.kt) * 7919u);
  }
};
int cached_weight_map(CUtensorMap* out, const void* B, int64_t n, int64_t kt) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{B, n, kt};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto f = cache.find(key);
    if (f != cache.end()) {
      *out = f->second;
      return UNIQL_OK;
    }
  }
  int st = make_weight_map(out, B, n, kt);
  if (st != UNIQL_OK) return st;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache[key] = *out;
  return UNIQL_OK;
}

struct DecodePlan {
  int variant;        // 0: 16 warps, three ring slots, m <= 2;  1: 16 warps, two slots, m <= 8;
                      // 2: 12 warps, two batch tiles (m <= 16);  3: 8 warps, two slots, m <= 8 (two launches fit an SM)
  int ring;
  int warps, grid, units;
  SlotGeom G;
  int fused_had;      // the Hadamard transform runs in the kernel prologue
  int hP, hlogP, hlogQ, hMdim, hbase, seg0;
  int xbytes;
  size_t smem;
  size_t partial_bytes;
};

static int ilog2(int64_t v) {
  int l = 0;
  while ((1ll << l) < v) ++l;
  return l;
}

// Geometry of a launch: depends on the shapes only (and on the SM count of the current device).
static int make_plan(DecodePlan* pl, int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue,
                     int64_t hadamard_dim, int64_t k_offset) {
  if (m < 1 || m > 16 || nproj < 1 || nproj > kMaxProj || k <= 0 || k % 128) return UNIQL_ESHAPE;
  DecodePlan P{};
  P.variant = m <= 2 ? 0 : m <= 8 ? 1 : 2;
  static const int force_variant = env_int("UNIQL_B200_DECODE_VARIANT", -1);
  if (force_variant == 3 && m <= 8) P.variant = 3;
  if (force_variant == 1 && m <= 8) P.variant = 1;
  P.warps = P.variant == 2 ? 12 : P.variant == 3 ? 8 : 16;
  P.ring = P.variant == 0 ? 3 : 2;
  P.grid = device_info().sm_count;
  P.G.W = P.grid * P.warps;
  P.G.NG = (int)(k / 128);
  int64_t vb = 0;
  for (int i = 0; i < nproj; ++i) {
    if (n[i] <= 0 || n[i] % 64) return UNIQL_ESHAPE;
    vb += n[i] / 64;
  }
  if (epilogue == UNIQL_EPILOGUE_SWIGLU && (nproj != 2 || n[0] != n[1])) return UNIQL_EINVAL;
  if (epilogue != UNIQL_EPILOGUE_NONE && epilogue != UNIQL_EPILOGUE_SWIGLU) return UNIQL_EINVAL;
  P.units = (int)(epilogue == UNIQL_EPILOGUE_SWIGLU ? vb / 2 : vb);
  if ((size_t)P.units * sizeof(int) > UNIQL_SCRATCH_COUNTER_BYTES) return UNIQL_ESHAPE;
  P.G.vbT = (int)vb;
  P.G.T = (long long)vb * P.G.NG;
  P.G.kc = P.G.NG; P.G.koff = 0; P.G.nchunks = 1;
  auto refresh = [&]() {
    P.G.dT = make_fastdiv((unsigned long long)P.G.T); P.G.dW = make_fastdiv((unsigned long long)P.G.W);
    P.G.dNG = make_fastdiv((unsigned long long)P.G.NG); P.G.dvbT = make_fastdiv((unsigned long long)P.G.vbT);
    P.G.dkc = make_fastdiv((unsigned long long)P.G.kc);
  };
  refresh();
  P.fused_had = 0;
  if (hadamard_dim) {
    const int base = hadamard_base_of(hadamard_dim);
    if (base == 0 || hadamard_dim > 40960 || k_offset < 0 || k_offset % 128 || k_offset + k > hadamard_dim) return UNIQL_ESHAPE;
    int64_t pw = hadamard_dim / base;             // power-of-two part
    int64_t seg = pw < 512 ? pw : 512;
    P.hP = (int)seg; P.hlogP = ilog2(seg); P.hlogQ = ilog2(pw / seg); P.hMdim = (int)(hadamard_dim / seg);
    P.hbase = base;
    // the prologue holds one transformed segment per 128-value group or more, batches of at most 4 rows, and a base
    // index that fits the 96-bit sign masks
    if (seg >= 128 && m <= 4 && P.hMdim <= 96 && env_int("UNIQL_B200_FUSED_HADAMARD", 1)) {
      P.G.kc = (int)(seg / 128);
      const int64_t g0 = k_offset / 128;
      P.G.koff = (int)(g0 % P.G.kc);
      P.seg0 = (int)(g0 / P.G.kc);
      P.G.nchunks = (P.G.NG + P.G.koff + P.G.kc - 1) / P.G.kc;
      refresh();
      // every CTA must touch at most kMaxSeg segments
      int worst = 0;
      for (int cta = 0; cta < P.grid; ++cta) {
        const long long a = warp_begin(P.G, cta * P.warps), b = warp_begin(P.G, (cta + 1) * P.warps);
        if (b <= a) continue;
        const int c0 = slot_decode(P.G, a).c, c1 = slot_decode(P.G, b - 1).c;
        if (c1 - c0 + 1 > worst) worst = c1 - c0 + 1;
      }
      if (worst <= kMaxSeg && P.G.nchunks <= 96) P.fused_had = 1;
      else { P.G.kc = P.G.NG; P.G.koff = 0; P.G.nchunks = 1; refresh(); }
    }
  }
  // tiles a block can receive per chunk
  int pc = 1;
  for (int cc = 0; cc < P.G.nchunks; ++cc) {
    const int lo = chunk_lo(cc, P.G.kc, P.G.koff), hi = chunk_hi(cc, P.G.kc, P.G.koff, P.G.NG);
    for (int b = 0; b < P.G.vbT; ++b) {
      const int r = runs_of(P.G, b, lo, hi);
      if (r > pc) pc = r;
    }
  }
  P.G.Pc = pc;
  P.partial_bytes = (size_t)P.G.vbT * P.G.nchunks * P.G.Pc * (size_t)m * 64 * sizeof(uint2);
  P.xbytes = P.fused_had ? 0 : (int)m * kXRowBytes;
  const size_t rings = (size_t)P.warps * P.ring * (kSlotBytes + kSlotScaleBytes);
  const size_t xs = P.fused_had ? (size_t)kMaxSeg * m * kSegRowBytes * (m == 1 ? 2 : 1) : (size_t)P.warps * P.ring * P.xbytes;
  P.smem = rings + xs;
  *pl = P;
  return UNIQL_OK;
}

struct PlanKey {
  int64_t m, k, n[kMaxProj], had, koff;
  int nproj, epilogue, dev;
  bool operator==(const PlanKey& o) const {
    if (m != o.m || k != o.k || had != o.had || koff != o.koff || nproj != o.nproj || epilogue != o.epilogue || dev != o.dev)
      return false;
    for (int i = 0; i < kMaxProj; ++i)
      if (n[i] != o.n[i]) return false;
    return true;
  }
};
struct PlanKeyHash {
  size_t operator()(const PlanKey& k) const {
    size_t h = (size_t)k.m * 1000003u ^ (size_t)k.k * 7919u ^ (size_t)k.had * 31u ^ (size_t)k.koff * 131u ^
               (size_t)k.nproj * 17u ^ (size_t)k.epilogue * 13u ^ (size_t)k.dev * 11u;
    for (int i = 0; i < kMaxProj; ++i) h = h * 1315423911u ^ (size_t)k.n[i];
    return h;
  }
};
static int cached_plan(DecodePlan* pl, int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue,
                       int64_t hadamard_dim, int64_t k_offset) {
  static std::mutex mu;
  static std::unordered_map<PlanKey, DecodePlan, PlanKeyHash> cache;
  PlanKey key{};
  key.m = m; key.k = k; key.had = hadamard_dim; key.koff = k_offset; key.nproj = nproj; key.epilogue = epilogue;
  cudaGetDevice(&key.dev);
  for (int i = 0; i < kMaxProj; ++i) key.n[i] = (i < nproj && nproj <= kMaxProj) ? n[i] : 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto f = cache.find(key);
    if (f != cache.end()) {
      *pl = f->second;
      return UNIQL_OK;
    }
  }
  int st = make_plan(pl, m, k, n, nproj, epilogue, hadamard_dim, k_offset);
  if (st != UNIQL_OK) return st;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *pl;
  return UNIQL_OK;
}

static inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

size_t decode_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue, int64_t hadamard_dim,
                            int64_t k_offset) {
  DecodePlan pl;
  if (cached_plan(&pl, m, k, n, nproj, epilogue, hadamard_dim, k_offset) != UNIQL_OK) return UNIQL_SCRATCH_COUNTER_BYTES;
  size_t total = UNIQL_SCRATCH_COUNTER_BYTES + align256(pl.partial_bytes);
  if (hadamard_dim && !pl.fused_had) total += align256((size_t)m * hadamard_dim * 2);   // separate transform kernel
  // whichever of the two decode kernels the launch ends up on
  size_t tiled = gemv_scratch_bytes(m, k, n, nproj, epilogue);
  if (hadamard_dim) tiled += align256((size_t)m * hadamard_dim * 2);
  return total > tiled ? total : tiled;
}

// Which decode kernel runs a launch.  The CTA-tiled kernel of w4a16_gemv.cu is the default: its reduction stays inside
// the CTA or the cluster and a launch costs about half as much; it also carries the tensor-parallel exchanges.
// UNIQL_B200_DECODE_ENGINE=slot selects the slot-balanced kernel of this file for single-GPU launches (tests,
// profiling); that kernel runs an online Hadamard transform in its own prologue.
static bool use_slot_engine(const DecodeArgs& a) {
  if (a.comm) return false;
  const char* e = getenv("UNIQL_B200_DECODE_ENGINE");
  return e && e[0] == 's';
}

template <int MT, int WARPS, int MINB, bool HAD, int RING>
static int launch_variant(const DecodeParams& p, const DecodePlan& pl, cudaStream_t stream) {
  auto kern = w4a16_decode_kernel<MT, WARPS, MINB, HAD, RING>;
  {
    // function attributes are per device; raise the dynamic shared-memory limit to what this launch needs
    static thread_local size_t attr_bytes[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (pl.smem > attr_bytes[dev]) {
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
      attr_bytes[dev] = pl.smem;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int nattr = 0;
  // Every launch may start early behind its predecessor; the kernel itself waits (griddepcontrol.wait)
  // before it touches anything another kernel could have written.
  static const int pdl_on = env_int("UNIQL_B200_PDL", 1);
  if (pdl_on) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  UNIQL_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return UNIQL_OK;
}

int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
  int64_t n[kMaxProj] = {0, 0, 0, 0};
  if (a.nproj < 1 || a.nproj > kMaxProj) return UNIQL_EINVAL;
  for (int i = 0; i < a.nproj; ++i) n[i] = a.proj[i].n;
  if (!use_slot_engine(a)) {
    // CTA-tiled kernel; an online Hadamard runs as its own kernel in front (rows rounded to fp16 in scratch) and the
    // linear's weight stream overlaps it through the programmatic dependent launch
    const size_t base = gemv_scratch_bytes(a.m, a.k, n, a.nproj, a.epilogue);
    const size_t xh_bytes = a.hadamard_dim ? align256((size_t)a.m * a.hadamard_dim * 2) : 0;
    if (!a.scratch || a.scratch_bytes < base + xh_bytes || (reinterpret_cast<uintptr_t>(a.scratch) & 255u)) return UNIQL_ESCRATCH;
    const __half* Ain = (const __half*)a.A;
    int64_t lda = a.lda;
    if (a.hadamard_dim) {
      __half* xh = (__half*)((char*)a.scratch + base);
      const float hscale = (float)(1.0 / sqrt((double)a.hadamard_dim));
      int st;
      if (a.comm && a.comm->gather_in) {
        // tensor parallel: the full row sits in this rank's feature area; every rank transforms it and multiplies
        // its own k slice of the result
        if (a.k_offset % 128 || a.k_offset + a.k > a.hadamard_dim) return UNIQL_ESHAPE;
        st = launch_hadamard_feat(*a.comm, xh, a.hadamard_dim, a.m, a.hadamard_dim, hscale, a.status_word, stream);
        Ain = xh + a.k_offset;
      } else {
        if (a.k_offset != 0 || a.k != a.hadamard_dim) return UNIQL_ESHAPE;
        st = launch_hadamard(a.A, a.lda, xh, a.hadamard_dim, a.m, a.hadamard_dim, hscale, UNIQL_F16, true, stream);
        Ain = xh;
      }
      if (st != UNIQL_OK) return st;
      lda = a.hadamard_dim;
    }
    return launch_gemv_group(a, Ain, lda, stream);
  }
  DecodePlan pl;
  int st = cached_plan(&pl, a.m, a.k, n, a.nproj, a.epilogue, a.hadamard_dim, a.k_offset);
  if (st != UNIQL_OK) return st;
  if (a.comm) return UNIQL_EINVAL;       // launches that talk to other GPUs run on the CTA-tiled kernel
  const size_t part_off = UNIQL_SCRATCH_COUNTER_BYTES;
  const size_t xh_off = part_off + align256(pl.partial_bytes);
  const size_t need = xh_off + ((a.hadamard_dim && !pl.fused_had) ? align256((size_t)a.m * a.hadamard_dim * 2) : 0);
  if (!a.scratch || a.scratch_bytes < need || (reinterpret_cast<uintptr_t>(a.scratch) & 255u)) return UNIQL_ESCRATCH;

  const __half* Ain = (const __half*)a.A;
  int64_t lda = a.lda;
  if (a.hadamard_dim && !pl.fused_had) {
    // separate transform kernel in front (rows of more than 4, or a split the prologue does not cover); the decode
    // kernel's weight stream overlaps it through the programmatic dependent launch
    if (a.k_offset != 0 || a.k != a.hadamard_dim) return UNIQL_ESHAPE;
    __half* xh = (__half*)((char*)a.scratch + xh_off);
    st = launch_hadamard(a.A, a.lda, xh, a.k, a.m, a.k, (float)(1.0 / sqrt((double)a.k)), UNIQL_F16, true, stream);
    if (st != UNIQL_OK) return st;
    Ain = xh;
    lda = a.k;
  }

  DecodeParams p;
  memset(&p, 0, sizeof(p));
  int vb = 0;
  for (int i = 0; i < a.nproj; ++i) {
    const DecodeProjArgs& q = a.proj[i];
    st = cached_weight_map(&p.wmap[i], q.B, q.n, a.k / 16);
    if (st != UNIQL_OK) return st;
    p.proj[i].S = (const __half*)q.s; p.proj[i].bias = (const __half*)q.bias; p.proj[i].D = (__half*)q.D;
    p.proj[i].ldd = q.ldd; p.proj[i].N = (int)q.n; p.proj[i].n_out = (int)q.n_out;
    p.vb_start[i] = vb;
    vb += (int)(q.n / 64);
  }
  for (int i = a.nproj; i <= kMaxProj; ++i) p.vb_start[i] = vb;
  for (int i = a.nproj; i < kMaxProj; ++i) { p.wmap[i] = p.wmap[0]; p.proj[i] = p.proj[0]; }
  p.A = Ain; p.lda = lda;
  p.residual = (const __half*)a.residual; p.ldr = a.ldr;
  p.partials = (uint2*)((char*)a.scratch + part_off);
  {
    // distinct per call where the host can tell calls apart; a captured launch replays with the same tag, which is
    // why consumers clear what they read
    static std::atomic<uint32_t> calls{0};
    p.tag = 1u + (calls.fetch_add(1, std::memory_order_relaxed) & 0x3fffffffu);
  }
  p.status_word = a.status_word;
  p.G = pl.G; p.M = (int)a.m; p.nproj = a.nproj; p.epilogue = a.epilogue;
  p.xbytes = pl.xbytes;
  p.had = pl.fused_had;
  if (pl.fused_had) {
    p.hP = pl.hP; p.hlogP = pl.hlogP; p.hlogQ = pl.hlogQ; p.hMdim = pl.hMdim; p.seg0 = pl.seg0;
    p.hscale = (float)(1.0 / sqrt((double)a.hadamard_dim));
    hadamard_base_signs(pl.hbase, p.hsign);
  }
  p.npf = 0;
  for (int i = 0; i < a.nprefetch && i < kMaxPrefetch; ++i)
    if (a.prefetch_ptr[i] && a.prefetch_bytes[i] >= 128) {
      p.pf_ptr[p.npf] = (const unsigned char*)a.prefetch_ptr[i];
      p.pf_lines[p.npf] = (long long)(a.prefetch_bytes[i] / 128);
      ++p.npf;
    }
  if (pl.fused_had) {
    if (pl.variant == 0) return launch_variant<1, 16, 1, true, 3>(p, pl, stream);
    if (pl.variant == 3) return launch_variant<1, 8, 2, true, 2>(p, pl, stream);
    return launch_variant<1, 16, 1, true, 2>(p, pl, stream);     // m <= 4 here
  }
  if (pl.variant == 0) return launch_variant<1, 16, 1, false, 3>(p, pl, stream);
  if (pl.variant == 1) return launch_variant<1, 16, 1, false, 2>(p, pl, stream);
  if (pl.variant == 3) return launch_variant<1, 8, 2, false, 2>(p, pl, stream);
  return launch_variant<2, 12, 1, false, 2>(p, pl, stream);
}

// Host-side replay of the kernel's work split for one launch geometry: walks every warp's slots with the kernel's own
// iterator and checks that each slot is taken exactly once, that every run of slots lands in its own tile below the
// reserved count, and that the tickets of every block add up to what the last arriver waits for.
template <bool CH>
static int replay_plan(const DecodePlan& pl, int epilogue) {
  const bool swiglu = epilogue == UNIQL_EPILOGUE_SWIGLU;
  std::unordered_map<long long, int> tiles;
  std::unordered_map<int, long long> tickets;
  std::unordered_map<long long, int> seen;
  const SlotGeom& G = pl.G;
  // the reciprocal divisions against plain ones
  for (int wg = 0; wg <= G.W; ++wg)
    if (warp_begin(G, wg) != G.T * wg / G.W) return 12;
  for (int wg = 0; wg < G.W; ++wg) {
    const long long s0 = warp_begin(G, wg), s1 = warp_begin(G, wg + 1);
    if (s1 <= s0) continue;
    if (warp_of_slot(G, s0) != wg || warp_of_slot(G, s1 - 1) != wg) return 1;
    if (warp_of_slot(G, s0) != (int)(((s0 + 1) * G.W - 1) / G.T)) return 13;
    SlotIt it = slot_at<CH>(G, s0);
    int run = 0;
    for (long long i = 0; i < s1 - s0; ++i) {
      const SlotIt ref = slot_decode(G, s0 + i);
      {
        // slot_decode itself against plain division
        const long long sl = s0 + i;
        const int q = (int)(sl / G.vbT), cpl = (q + G.koff) / G.kc;
        if (ref.c != cpl) return 14;
      }
      if (ref.vb != it.vb || ref.g != it.g || ref.c != it.c || ref.g_lo != it.g_lo || ref.g_hi != it.g_hi) return 2;
      if (it.vb < 0 || it.vb >= G.vbT || it.g < 0 || it.g >= G.NG) return 3;
      const long long id = (long long)it.vb * G.NG + it.g;
      if (seen[id]++) return 4;
      ++run;
      if (i == s1 - s0 - 1 || it.g + 1 == it.g_hi) {
        const int wc = it.g_hi - it.g_lo;
        const long long first = (long long)G.vbT * it.g_lo + (long long)it.vb * wc;
        const int jrun = run_index(G, first, s0 + i - (run - 1), wg);
        if (jrun < 0 || jrun >= G.Pc || it.c < 0 || it.c >= G.nchunks) return 5;
        if (jrun >= runs_of(G, it.vb, it.g_lo, it.g_hi)) return 6;
        const long long tile = ((long long)it.vb * G.nchunks + it.c) * G.Pc + jrun;
        if (tiles[tile]++) return 7;
        tickets[swiglu ? it.vb >> 1 : it.vb] += run;
        run = 0;
      }
      slot_next<CH>(G, it);
    }
  }
  if ((long long)seen.size() != G.T) return 8;
  if ((int)tickets.size() != pl.units) return 9;
  for (auto& kv : tickets)
    if (kv.second != (swiglu ? 2 : 1) * (long long)G.NG) return 10;
  // the number of tiles a block's finisher reads equals the number written
  long long expect = 0;
  for (int cc = 0; cc < G.nchunks; ++cc)
    for (int b = 0; b < G.vbT; ++b)
      expect += runs_of(G, b, chunk_lo(cc, G.kc, G.koff), chunk_hi(cc, G.kc, G.koff, G.NG));
  if (expect != (long long)tiles.size()) return 11;
  return 0;
}

// ------------------------------------------------------------------ entry point without allocation
// Scratch for uniql_w4a16_linear_static: ticket counters followed by the partial tiles.  It lives in the
// library image: every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[UNIQL_STATIC_SCRATCH_BYTES];

struct StaticScratchState {
  void* ptr;      // device address of g_static_scratch on that device
  bool ready;
};
static StaticScratchState g_static_state[64];
static std::mutex g_static_mutex;

// Resolves the device address of the array (its name is only a host-side handle) once per device, with that
// device current, and clears the counter region through the caller's stream.
static int static_scratch_for_current_device(void** out, cudaStream_t stream) {
  int dev = 0;
  UNIQL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return UNIQL_EINVAL;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticScratchState& st = g_static_state[dev];
  if (!st.ready) {
    void* ptr = nullptr;
    UNIQL_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    UNIQL_CUDA_TRY(cudaMemsetAsync(ptr, 0, UNIQL_SCRATCH_COUNTER_BYTES, stream));
    st.ptr = ptr;
    st.ready = true;
  }
  *out = st.ptr;
  return UNIQL_OK;
}

}  // namespace uniql

extern "C" int uniql_w4a16_plan_selftest(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue,
                                         int64_t hadamard_dim, int64_t k_offset, int* fused_hadamard_out) {
  using namespace uniql;
  if (!n) return UNIQL_EINVAL;
  DecodePlan pl;
  int st = make_plan(&pl, m, k, n, nproj, epilogue, hadamard_dim, k_offset);
  if (st != UNIQL_OK) return st;
  if (fused_hadamard_out) *fused_hadamard_out = pl.fused_had;
  return pl.fused_had ? replay_plan<true>(pl, epilogue) : replay_plan<false>(pl, epilogue);
}

extern "C" int uniql_w4a16_linear_static(const void* A, int64_t lda, const void* B, const void* s, const void* bias,
                                         void* D, int64_t ldd, int64_t m, int64_t n, int64_t n_out, int64_t k,
                                         int groupsize, int* status_word, void* stream_) {
  using namespace uniql;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (groupsize != 128) return groupsize == -1 ? UNIQL_EGROUPSIZE : UNIQL_EINVAL;
  if (m < 0 || n <= 0 || k <= 0 || n_out <= 0 || n_out > n) return UNIQL_EINVAL;
  if (m > 16) return UNIQL_ESHAPE;                       // decode kernel only
  if (n % 64 != 0 || k % 128 != 0 || n > (int64_t)1 << 22 || k > (int64_t)1 << 22) return UNIQL_ESHAPE;
  if (lda < k || ldd < n_out || lda % 8 != 0) return UNIQL_EINVAL;
  if (m == 0) return UNIQL_OK;
  if (!A || !B || !s || !D) return UNIQL_EINVAL;
  if (!aligned16(A) || !aligned16(B) || !aligned16(s) || (reinterpret_cast<uintptr_t>(D) & 1u)) return UNIQL_EINVAL;
  // the figure uniql_w4a16_scratch_bytes reports for the problem (what either decode kernel would need)
  const size_t need = decode_scratch_bytes(m, k, &n, 1, UNIQL_EPILOGUE_NONE, 0, 0);
  if (need > (size_t)UNIQL_STATIC_SCRATCH_BYTES) return UNIQL_ESTATIC;
  void* scratch = nullptr;
  int st = static_scratch_for_current_device(&scratch, stream);
  if (st != UNIQL_OK) return st;
  DecodeArgs a{};
  a.A = A; a.lda = lda; a.m = m; a.k = k; a.nproj = 1;
  a.proj[0].B = B; a.proj[0].s = s; a.proj[0].bias = bias; a.proj[0].D = D; a.proj[0].ldd = ldd;
  a.proj[0].n = n; a.proj[0].n_out = n_out;
  a.epilogue = UNIQL_EPILOGUE_NONE;
  a.scratch = scratch; a.scratch_bytes = UNIQL_STATIC_SCRATCH_BYTES;
  a.status_word = status_word;
  a.comm = nullptr;
  a.nprefetch = 0;
  return launch_decode(a, stream);
}
