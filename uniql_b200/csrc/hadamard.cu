// Hadamard transform along the last axis for sm_100a:  y = (H_base (x) H_{2^j}) x * scale.
//
// Replaces the third-party fast_hadamard_transform_cuda entry points UniQL calls from
// quantize/hadamard_helpers.py:18-48 (power-of-two, 12N, 20N, 28N, 40N).  The index splits as
// i = a * 2^j + b: b runs through a Sylvester-ordered Walsh-Hadamard transform, a through a fixed
// base x base Hadamard matrix (Paley I for 12 and 20, Paley II for 28, H_2 (x) H_20 for 40).
//
// Many rows of a 16-bit type with 128 <= P <= 512: hadamard_mma_kernel -- the base matrix (or H_16 / H_32 for a
// power-of-two size) is applied first, to the raw inputs, as an mma.sync with a +1/-1 operand; the P-point part follows
// in fp32; persistent CTAs prefetch the next row while they work (see the comment at the kernel).
// Other many-row cases: one CTA per row.  hadamard_rows32_kernel (P >= 32): each thread takes 32 contiguous elements (four
// 16-byte loads for 16-bit types), does 5 butterfly stages in registers and parks the result in a padded fp32 copy in
// shared memory; the remaining stages run radix-8/4/2 out of shared memory (stride >= 32, bank-conflict free); the base
// matrix is applied per column b with compile-time signs, scaled, converted and stored coalesced.  hadamard_kernel
// (tiny transforms): 8 contiguous elements per thread, 3 register stages and up to 5 shuffle stages.
// Few rows (decode): hadamard_split_kernel, one CTA per (segment, row); hadamard_split_feat_kernel reads the row from a
// tensor-parallel layer's feature area.  A base matrix replaced at run time (uniql_hadamard_set_base_matrix) is honoured
// by every path (hadamard_rt_kernel where the signs are otherwise compiled in).
// HBM-bound for many rows (2 * dim * sizeof(T) bytes per row); latency-bound for a single row.
#include "common.cuh"
#include "linear_internal.cuh"

#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <type_traits>
#include <utility>

namespace uniql {

struct HadSigns {
  uint64_t row[64];   // bit a' of row[a] set  <=>  H[a][a'] = -1
};

// ------------------------------------------------------------- base matrices (deterministic, one definition)
// Paley I for 12 and 20, Paley II for 28, H_2 (x) H_20 for 40, element by element as constexpr functions: the host
// uses them to fill sign masks and the exported matrix, the row kernel instantiates them at compile time so that its
// base pass is plain FADD / FSUB with the signs folded into the instructions (a sign mask read at run time costs an
// extra XOR per term and made that pass three quarters of the kernel's instructions).
__host__ __device__ constexpr int c_legendre(int a, int q) {
  a %= q;
  if (a < 0) a += q;
  if (a == 0) return 0;
  long long r = 1, b = a;
  int e = (q - 1) / 2;
  while (e) {
    if (e & 1) r = r * b % q;
    b = b * b % q;
    e >>= 1;
  }
  return r == 1 ? 1 : -1;
}
__host__ __device__ constexpr int c_paley1(int q, int i, int j) {
  int v = 0;
  if (i == 0 && j == 0) v = 0;
  else if (i == 0) v = 1;
  else if (j == 0) v = -1;
  else v = c_legendre(j - i, q);
  if (i == j) v += 1;
  return v;
}
__host__ __device__ constexpr int c_paley2(int q, int r, int c) {
  const int i = r >> 1, j = c >> 1, n = q + 1;
  (void)n;
  int cij = 0;
  if (i == 0 && j == 0) cij = 0;
  else if (i == 0 || j == 0) cij = 1;
  else cij = c_legendre(j - i, q);
  const int pos = (r & 1) * 2 + (c & 1);
  if (cij == 0) return pos == 3 ? -1 : 1;
  return pos == 0 ? cij : -cij;
}
__host__ __device__ constexpr int c_base_entry(int base, int i, int j) {
  if (base == 12) return c_paley1(11, i, j);
  if (base == 20) return c_paley1(19, i, j);
  if (base == 28) return c_paley2(13, i, j);
  // 40: H_2 (x) H_20
  const int v = c_paley1(19, i % 20, j % 20);
  return (i >= 20 && j >= 20) ? -v : v;
}

// A caller may replace a base matrix at run time (uniql_hadamard_set_base_matrix): whoever holds the matrices of the
// third-party package the reference links can make every transform of this library use them without a rebuild.  The
// few-row kernels and the linear kernel's prologue take their signs as launch parameters and follow at full speed;
// the many-row kernels have the built-in signs compiled in, so sizes of a replaced order go to hadamard_rt_kernel.
static std::mutex g_base_mu;
static bool g_base_custom[4] = {false, false, false, false};
static int8_t g_base_h[4][1600];
static unsigned g_base_generation = 0;       // bumped by every replacement; host-side sign caches compare it

struct BuiltinBases {
  int8_t h[4][1600];
  BuiltinBases() {
    const int orders[4] = {12, 20, 28, 40};
    for (int s = 0; s < 4; ++s)
      for (int i = 0; i < orders[s]; ++i)
        for (int j = 0; j < orders[s]; ++j) h[s][i * orders[s] + j] = (int8_t)c_base_entry(orders[s], i, j);
  }
};
static const BuiltinBases& builtin_bases() {
  static const BuiltinBases b;
  return b;
}
static int base_slot(int base) { return base == 12 ? 0 : base == 20 ? 1 : base == 28 ? 2 : base == 40 ? 3 : -1; }

static bool base_is_custom(int base) {
  const int s = base_slot(base);
  if (s < 0) return false;
  std::lock_guard<std::mutex> lk(g_base_mu);
  return g_base_custom[s];
}

static int base_matrix(int base, int8_t* h) {
  const int s = base_slot(base);
  if (s < 0) return UNIQL_ESHAPE;
  {
    std::lock_guard<std::mutex> lk(g_base_mu);
    if (g_base_custom[s]) {
      for (int i = 0; i < base * base; ++i) h[i] = g_base_h[s][i];
      return UNIQL_OK;
    }
  }
  memcpy(h, builtin_bases().h[s], (size_t)base * base);
  return UNIQL_OK;
}

static int set_base_matrix(int base, const int8_t* h) {
  const int s = base_slot(base);
  if (s < 0) return UNIQL_ESHAPE;
  if (h) {
    for (int i = 0; i < base * base; ++i)
      if (h[i] != 1 && h[i] != -1) return UNIQL_EINVAL;
    for (int i = 0; i < base; ++i)
      for (int j = 0; j < base; ++j) {
        int dot = 0;
        for (int t = 0; t < base; ++t) dot += h[i * base + t] * h[j * base + t];
        if (dot != (i == j ? base : 0)) return UNIQL_EINVAL;      // rows must be orthogonal: H H^T = base I
      }
  }
  std::lock_guard<std::mutex> lk(g_base_mu);
  g_base_custom[s] = h != nullptr;
  if (h)
    for (int i = 0; i < base * base; ++i) g_base_h[s][i] = h[i];
  ++g_base_generation;
  return UNIQL_OK;
}

void hadamard_base_signs(int base, unsigned long long* rows40) {
  for (int i = 0; i < 40; ++i) rows40[i] = 0ull;
  int8_t h[1600];
  if (base_matrix(base, h) != UNIQL_OK) return;
  for (int i = 0; i < base; ++i)
    for (int j = 0; j < base; ++j)
      if (h[i * base + j] < 0) rows40[i] |= (1ull << j);
}

static bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

int hadamard_base_of(int64_t dim) {
  if (dim <= 0) return 0;
  const int bases[4] = {40, 28, 20, 12};   // the reference's dispatch order
  for (int b : bases)
    if (dim % b == 0 && is_pow2(dim / b)) return b;
  return is_pow2(dim) ? 1 : 0;
}

// ------------------------------------------------------------- element access
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static __device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), v);
  }
  static __device__ __forceinline__ void store8(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), v);
  }
  static __device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ void unpack8(const uint4&, float (&)[8]) {}   // 16-bit types only
  static __device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  static __device__ __forceinline__ void store1(float* p, float v) { *p = v; }
};

template <int R>
__device__ __forceinline__ void butterflies(float (&v)[R]) {
#pragma unroll
  for (int s = 1; s < R; s <<= 1)
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (!(i & s)) {
        const float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
}

template <int R>
__device__ __forceinline__ void strided_pass(float* buf, int dim, int h, int tid, int nthreads) {
  const int groups = dim / R;
  const int lh = __ffs(h) - 1;                  // h is a power of two: shifts and masks instead of divisions
  for (int idx = tid; idx < groups; idx += nthreads) {
    const int low = idx & (h - 1), high = idx >> lh;
    float* p = buf + (size_t)high * h * R + low;
    float v[R];
#pragma unroll
    for (int i = 0; i < R; ++i) v[i] = p[(size_t)i * h];
    butterflies<R>(v);
#pragma unroll
    for (int i = 0; i < R; ++i) p[(size_t)i * h] = v[i];
  }
}

// Padded shared-memory layout of the 32-element kernel: 4 floats of padding after every 32, so that lanes storing
// their 32 contiguous elements as 16-byte vectors (lane stride 144 bytes) hit distinct banks.
__device__ __forceinline__ int pad32(int e) { return e + ((e >> 5) << 2); }

template <int R>
__device__ __forceinline__ void strided_pass_padded(float* buf, int total, int h, int tid, int nthreads) {
  const int groups = total / R;
  const int hp = h + (h >> 3);                  // pad32 is linear in steps of h when h is a multiple of 32
  const int lh = __ffs(h) - 1;                  // h is a power of two: shifts and masks instead of divisions
  for (int idx = tid; idx < groups; idx += nthreads) {
    const int low = idx & (h - 1), high = idx >> lh;
    float* p = buf + pad32(high * h * R + low);
    float v[R];
#pragma unroll
    for (int i = 0; i < R; ++i) v[i] = p[(size_t)i * hp];
    butterflies<R>(v);
#pragma unroll
    for (int i = 0; i < R; ++i) p[(size_t)i * hp] = v[i];
  }
}

template <int BASE, int A, size_t... I>
__device__ __forceinline__ float base_row(const float (&z)[BASE], std::index_sequence<I...>) {
  return ((std::integral_constant<int, c_base_entry(BASE, A, (int)I)>::value > 0 ? z[I] : -z[I]) + ...);
}
// ALL: the thread writes every output row of its column (no range test, no branches around the stores).
template <typename T, bool ALL>
__device__ __forceinline__ void put_row(T* dst, int a, int P, int a_lo, int a_hi, float v) {
  if (ALL || (a >= a_lo && a < a_hi)) Elem<T>::store1(dst + (size_t)a * P, v);
}
template <typename T, int BASE, bool ALL, size_t... A>
__device__ __forceinline__ void base_rows(const float (&z)[BASE], T* dst, int P, int a_lo, int a_hi, float scale,
                                          std::index_sequence<A...>) {
  (put_row<T, ALL>(dst, (int)A, P, a_lo, a_hi, base_row<BASE, (int)A>(z, std::make_index_sequence<BASE>{}) * scale), ...);
}
// Order-28 matrix (Paley II over GF(13)) through its 2 x 2 block structure: with u_j = z_2j - z_2j+1 and
// v_j = -(z_2j + z_2j+1), rows 2i and 2i+1 are  sum_{j != i} c_ij u_j - v_i  and  sum_{j != i} c_ij v_j + u_i
// where c is the 14 x 14 symmetric core (c_ij = 1 on the border, else the Legendre symbol of j - i): 392 adds per
// column instead of 756.
__host__ __device__ constexpr int c_core14(int i, int j) {
  return (i == 0 || j == 0) ? 1 : c_legendre(j - i, 13);
}
template <int I, int J>
__device__ __forceinline__ float core14_acc(const float (&w)[14], float acc) {
  if constexpr (J == 14) return acc;
  else if constexpr (J == I) return core14_acc<I, J + 1>(w, acc);
  else return core14_acc<I, J + 1>(w, std::integral_constant<int, c_core14(I, J)>::value > 0 ? acc + w[J] : acc - w[J]);
}
template <typename T, bool ALL, size_t... I>
__device__ __forceinline__ void base_rows28(const float (&u)[14], const float (&v)[14], T* dst, int P, int a_lo, int a_hi,
                                            float scale, std::index_sequence<I...>) {
  (put_row<T, ALL>(dst, (int)(2 * I), P, a_lo, a_hi, core14_acc<(int)I, 0>(u, -v[I]) * scale), ...);
  (put_row<T, ALL>(dst, (int)(2 * I + 1), P, a_lo, a_hi, core14_acc<(int)I, 0>(v, u[I]) * scale), ...);
}
template <typename T, bool ALL, size_t... A>
__device__ __forceinline__ void base_rows40(const float (&sm)[20], const float (&df)[20], T* dst, int P, int a_lo, int a_hi,
                                            float scale, std::index_sequence<A...>) {
  (put_row<T, ALL>(dst, (int)A, P, a_lo, a_hi, base_row<20, (int)A>(sm, std::make_index_sequence<20>{}) * scale), ...);
  (put_row<T, ALL>(dst, (int)(20 + A), P, a_lo, a_hi, base_row<20, (int)A>(df, std::make_index_sequence<20>{}) * scale), ...);
}
template <typename T, int BASE, bool ALL>
__device__ __forceinline__ void base_column(const float (&z)[BASE], T* dst, int P, int a_lo, int a_hi, float scale) {
  if constexpr (BASE == 28) {
    float u[14], v[14];
#pragma unroll
    for (int j = 0; j < 14; ++j) { u[j] = z[2 * j] - z[2 * j + 1]; v[j] = -z[2 * j] - z[2 * j + 1]; }
    base_rows28<T, ALL>(u, v, dst, P, a_lo, a_hi, scale, std::make_index_sequence<14>{});
  } else if constexpr (BASE == 40) {
    // H_40 = [[H_20, H_20], [H_20, -H_20]]: two order-20 products of the sum and the difference of the halves
    float sm[20], df[20];
#pragma unroll
    for (int j = 0; j < 20; ++j) { sm[j] = z[j] + z[20 + j]; df[j] = z[j] - z[20 + j]; }
    base_rows40<T, ALL>(sm, df, dst, P, a_lo, a_hi, scale, std::make_index_sequence<20>{});
  } else {
    base_rows<T, BASE, ALL>(z, dst, P, a_lo, a_hi, scale, std::make_index_sequence<BASE>{});
  }
}
// Pass C of the row kernels: y[a * P + b] = scale * sum_a' H[a][a'] z[a' * P + b] for every column b.
template <typename T, int BASE, bool PAD = false>
__device__ __forceinline__ void base_pass(const float* buf, T* yr, int P, float scale, int tid, int nthreads) {
  int asplit = nthreads / P;            // spread the output rows of a column over idle threads
  if (asplit < 1) asplit = 1;
  if (asplit > 8) asplit = 8;
  // distance between the segments of a column in the (padded) copy: pad32 is linear in steps of P (P % 32 == 0)
  const int seg_stride = PAD ? P + (P >> 3) : P;
  if (asplit == 1) {
    for (int b = tid; b < P; b += nthreads) {
      const float* col = buf + (PAD ? pad32(b) : b);
      float z[BASE];
#pragma unroll
      for (int a = 0; a < BASE; ++a) z[a] = col[(size_t)a * seg_stride];
      base_column<T, BASE, true>(z, yr + b, P, 0, BASE, scale);
    }
    return;
  }
  const int tasks = P * asplit;
  const int lp = __ffs(P) - 1;                  // P is a power of two
  for (int task = tid; task < tasks; task += nthreads) {
    const int b = task & (P - 1), part = task >> lp;
    const int a_lo = BASE * part / asplit, a_hi = BASE * (part + 1) / asplit;
    const float* col = buf + (PAD ? pad32(b) : b);
    float z[BASE];
#pragma unroll
    for (int a = 0; a < BASE; ++a) z[a] = col[(size_t)a * seg_stride];
    base_column<T, BASE, false>(z, yr + b, P, a_lo, a_hi, scale);
  }
}

template <typename T>
__global__ void __launch_bounds__(512) hadamard_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y,
                                                       int64_t ldy, int64_t rows, int rows_per_cta, int dim, int P,
                                                       int base, float scale, int pdl_trigger) {
  extern __shared__ __align__(16) float buf[];
  if (pdl_trigger) pdl_launch_dependents();   // the dependent kernel only prefetches until it waits on us
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31;
  // a CTA takes rows_per_cta consecutive rows (more than one for short rows, so that every thread has several
  // independent 16-byte loads in flight before the butterfly chain starts)
  const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
  const int nr = (int)(rows - row0 < rows_per_cta ? rows - row0 : rows_per_cta);
  const T* xr = x + row0 * ldx;
  T* yr = y + row0 * ldy;

  // ---- pass A: 8 contiguous elements per thread, stages h = 1..128 (limited by P) ----
  const int nchunks = dim >> 3;
  const int nchunks_pad = (nchunks + 31) & ~31;   // whole warps per row: the shuffle stages stay inside one row
  const int total = nr * nchunks_pad;
  const bool only_a = (base == 1 && P <= 256);   // whole transform fits pass A: store straight from registers
  constexpr int LB = 4;                          // chunks loaded together per thread
  for (int i0 = tid; i0 < total; i0 += nthreads * LB) {
    float v[LB][8];
    int row_of[LB], ch_of[LB];
#pragma unroll
    for (int u = 0; u < LB; ++u) {
      const int idx = i0 + u * nthreads;
      row_of[u] = idx / nchunks_pad;
      ch_of[u] = idx - row_of[u] * nchunks_pad;
      if (idx < total && ch_of[u] < nchunks) Elem<T>::load8(xr + (int64_t)row_of[u] * ldx + (size_t)ch_of[u] * 8, v[u]);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < LB; ++u) {
      if (i0 + u * nthreads >= total) break;     // uniform per warp: total and nthreads are multiples of 32
      butterflies<8>(v[u]);
#pragma unroll
      for (int s = 0; s < 5; ++s) {
        if ((8 << s) < P) {
          const bool upper = (lane >> s) & 1;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float o = __shfl_xor_sync(0xffffffffu, v[u][i], 1 << s);
            v[u][i] = upper ? (o - v[u][i]) : (v[u][i] + o);
          }
        }
      }
      if (ch_of[u] < nchunks) {
        if (only_a) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[u][i] *= scale;
          Elem<T>::store8(yr + (int64_t)row_of[u] * ldy + (size_t)ch_of[u] * 8, v[u]);
        } else {
          float4* d = reinterpret_cast<float4*>(buf + (size_t)row_of[u] * dim + (size_t)ch_of[u] * 8);
          d[0] = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
          d[1] = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
        }
      }
    }
  }
  if (only_a) return;
  __syncthreads();

  // ---- pass B: stages h = 256 .. P/2 out of shared memory (all rows of the CTA as one array: P divides dim) ----
  for (int h = 256; h < P;) {
    const int rem = P / h;
    if (rem >= 8) { strided_pass<8>(buf, nr * dim, h, tid, nthreads); h *= 8; }
    else if (rem == 4) { strided_pass<4>(buf, nr * dim, h, tid, nthreads); h *= 4; }
    else { strided_pass<2>(buf, nr * dim, h, tid, nthreads); h *= 2; }
    __syncthreads();
  }

  // ---- pass C: base matrix across the `base` segments, scale, store ----
  if (base == 1) {
    for (int idx = tid; idx < nr * nchunks; idx += nthreads) {
      const int r = idx / nchunks, ch = idx - r * nchunks;
      float v[8];
      const float4* s4 = reinterpret_cast<const float4*>(buf + (size_t)r * dim + (size_t)ch * 8);
      const float4 a = s4[0], b = s4[1];
      v[0] = a.x * scale; v[1] = a.y * scale; v[2] = a.z * scale; v[3] = a.w * scale;
      v[4] = b.x * scale; v[5] = b.y * scale; v[6] = b.z * scale; v[7] = b.w * scale;
      Elem<T>::store8(yr + (int64_t)r * ldy + (size_t)ch * 8, v);
    }
    return;
  }
  for (int r = 0; r < nr; ++r) {
    const float* rb = buf + (size_t)r * dim;
    T* ry = yr + (int64_t)r * ldy;
    if (base == 12) base_pass<T, 12>(rb, ry, P, scale, tid, nthreads);
    else if (base == 20) base_pass<T, 20>(rb, ry, P, scale, tid, nthreads);
    else if (base == 28) base_pass<T, 28>(rb, ry, P, scale, tid, nthreads);
    else base_pass<T, 40>(rb, ry, P, scale, tid, nthreads);
  }
}

// Many rows, P >= 32: one CTA per row, 32 contiguous elements per thread.  Stages h = 1..16 run in registers (no
// shuffles: the five shuffle stages of the 8-element kernel were most of its instructions), the rest as radix-8/4/2
// passes over the padded shared-memory copy, then the base matrix.
template <typename T>
__global__ void __launch_bounds__(256) hadamard_rows32_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y,
                                                              int64_t ldy, int dim, int P, int base, float scale,
                                                              int pdl_trigger) {
  extern __shared__ __align__(16) float buf[];
  if (pdl_trigger) pdl_launch_dependents();
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const T* xr = x + (int64_t)blockIdx.x * ldx;
  T* yr = y + (int64_t)blockIdx.x * ldy;
  const int nch = dim >> 5;

  for (int c = tid; c < nch; c += nthreads) {
    float v[32];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float t8[8];
      Elem<T>::load8(xr + (size_t)c * 32 + q * 8, t8);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[q * 8 + i] = t8[i];
    }
    butterflies<32>(v);
    float4* d = reinterpret_cast<float4*>(buf + c * 36);
#pragma unroll
    for (int q = 0; q < 8; ++q) d[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
  __syncthreads();

  for (int h = 32; h < P;) {
    const int rem = P / h;
    if (rem >= 8) { strided_pass_padded<8>(buf, dim, h, tid, nthreads); h *= 8; }
    else if (rem == 4) { strided_pass_padded<4>(buf, dim, h, tid, nthreads); h *= 4; }
    else { strided_pass_padded<2>(buf, dim, h, tid, nthreads); h *= 2; }
    __syncthreads();
  }

  if (base == 1) {
    for (int c = tid; c < nch * 4; c += nthreads) {     // 8 elements per step: never across a padding gap
      float v[8];
      const float4* s4 = reinterpret_cast<const float4*>(buf + pad32(c * 8));
      const float4 a = s4[0], b = s4[1];
      v[0] = a.x * scale; v[1] = a.y * scale; v[2] = a.z * scale; v[3] = a.w * scale;
      v[4] = b.x * scale; v[5] = b.y * scale; v[6] = b.z * scale; v[7] = b.w * scale;
      Elem<T>::store8(yr + (size_t)c * 8, v);
    }
    return;
  }
  if (base == 12) base_pass<T, 12, true>(buf, yr, P, scale, tid, nthreads);
  else if (base == 20) base_pass<T, 20, true>(buf, yr, P, scale, tid, nthreads);
  else if (base == 28) base_pass<T, 28, true>(buf, yr, P, scale, tid, nthreads);
  else base_pass<T, 40, true>(buf, yr, P, scale, tid, nthreads);
}

// Many rows with a base matrix given at run time: one CTA per row, the row as fp32 in shared memory, radix-2 passes
// over the power-of-two part, then per column b the base x base signed sums with the signs read from the launch
// parameters.  Plain and a few times slower than the kernels with compiled-in signs; it exists so that a replaced
// base matrix is honoured at every size.
template <typename T>
__global__ void __launch_bounds__(256) hadamard_rt_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y,
                                                          int64_t ldy, int dim, int P, int base, float scale,
                                                          const HadSigns signs, int pdl_trigger) {
  extern __shared__ __align__(16) float rt_buf[];
  if (pdl_trigger) pdl_launch_dependents();
  const int tid = threadIdx.x, nt = blockDim.x;
  const T* xr = x + (int64_t)blockIdx.x * ldx;
  T* yr = y + (int64_t)blockIdx.x * ldy;
  for (int c = tid; c < dim / 8; c += nt) {
    float t[8];
    Elem<T>::load8(xr + (size_t)c * 8, t);
#pragma unroll
    for (int e = 0; e < 8; ++e) rt_buf[c * 8 + e] = t[e];
  }
  __syncthreads();
  for (int h = 1; h < P; h <<= 1) {
    for (int idx = tid; idx < dim / 2; idx += nt) {
      const int i = (idx / h) * 2 * h + (idx % h);
      const float a = rt_buf[i], b = rt_buf[i + h];
      rt_buf[i] = a + b;
      rt_buf[i + h] = a - b;
    }
    __syncthreads();
  }
  for (int b = tid; b < P; b += nt) {
    float v[40];
#pragma unroll
    for (int a = 0; a < 40; ++a) v[a] = a < base ? rt_buf[(size_t)a * P + b] : 0.f;
    for (int ap = 0; ap < base; ++ap) {
      const uint64_t mask = signs.row[ap];
      float acc = 0.f;
#pragma unroll
      for (int a = 0; a < 40; ++a) acc += ((mask >> a) & 1ull) ? -v[a] : v[a];
      rt_buf[(size_t)ap * P + b] = acc * scale;      // column b belongs to this thread alone
    }
  }
  __syncthreads();
  for (int c = tid; c < dim / 8; c += nt) {
    float t[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) t[e] = rt_buf[c * 8 + e];
    Elem<T>::store8(yr + (size_t)c * 8, t);
  }
}

// Many rows of a 16-bit type, 128 <= P <= 512: the base matrix runs on the tensor cores.  The two factors of
// (H_base (x) H_P) commute, so the base matrix is applied FIRST, to the raw inputs: Z[a', b] = sum_a H[a'][a] X[a, b] is
// a matrix product with a +1/-1 operand -- exact products, fp32 sums -- and costs one mma.sync per 16 x 8 outputs instead
// of `base` adds per output (28 x 28 signed sums per column were three quarters of the row kernel's instructions).
// Power-of-two sizes use H_16 or H_32 in Sylvester order as their "base".  One CTA per row:
//   1. cp.async the row into shared memory as [a][b] (row stride P + 8 elements, so ldmatrix is conflict free);
//   2. warp (m-tile, 128-column unit): ldmatrix.trans gives the [k = a][n = b] operand, H sits in registers as the
//      16-row operand (signs from the launch parameters: a matrix replaced at run time costs nothing), 16 n-tiles ->
//      64 fp32 accumulators per thread; butterflies over the b bits a thread holds (0 and 3..6) in registers;
//   3. fp32 tile to shared memory (it reuses the raw row's space), second pass: a thread takes 8 consecutive b for every
//      128-column unit, runs bits 1, 2 and 7.., scales, converts and stores 16 bytes, coalesced.
template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  static constexpr unsigned kOne = 0x3C00u, kMinusOne = 0xBC00u;
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static constexpr unsigned kOne = 0x3F80u, kMinusOne = 0xBF80u;
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ uint32_t had_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void had_cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(had_smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

template <typename T, int MT, int LOGP>
__global__ void __launch_bounds__(MT * (1 << (LOGP - 7)) * 32, (MT == 3 && LOGP == 9) ? 1 : 2)
    hadamard_mma_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t ldy, int64_t rows, int base,
                        float scale, const HadSigns signs, int pdl_trigger) {
  constexpr int KT = MT;
  constexpr int P = 1 << LOGP;
  constexpr int NU = P / 128;
  constexpr int NTHREADS = MT * NU * 32;
  constexpr int RS = P + 8;     // row stride of the raw row (16-bit elements) and of the fp32 tile (words); 8 mod 32
  // Shared memory: three regions of base * RS * 2 bytes.  The raw row of iteration i sits in region c = 2 i mod 3; its
  // fp32 tile (twice the size) takes regions c and c + 1 -- rows a' < base / 2 in the first, the rest in the second;
  // the next row is fetched into region c + 2 while this one is worked on.
  extern __shared__ __align__(16) unsigned char had_smem[];
  const int region_bytes = base * RS * 2;
  const int half_rows = base >> 1;
  if (pdl_trigger) pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;

  // H as the 16-row operand (rows a', k = a), zero outside base x base: built once per CTA
  const int mt = warp % MT, u = warp / MT;
  uint32_t afrag[KT][4];
#pragma unroll
  for (int kt = 0; kt < KT; ++kt)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = 16 * mt + g + (j & 1) * 8;
      const int k = 16 * kt + 2 * c + (j >> 1) * 8;
      uint32_t w = 0;
      if (r < base) {
        const uint64_t m = signs.row[r];
        if (k < base) w |= ((m >> k) & 1ull) ? MmaOp<T>::kMinusOne : MmaOp<T>::kOne;
        if (k + 1 < base) w |= (((m >> (k + 1)) & 1ull) ? MmaOp<T>::kMinusOne : MmaOp<T>::kOne) << 16;
      }
      afrag[kt][j] = w;
    }
  // ldmatrix row of this lane: k = lane (and 32 + lane % 16 for a third k-tile); rows past `base` read row 0, whose
  // products meet the zero columns of H
  int k0 = KT == 1 ? (lane & 15) : lane;
  if (k0 >= base) k0 = 0;
  int k1 = 32 + (lane & 15);
  if (k1 >= base) k1 = 0;
  const uint32_t smem0 = had_smem_addr(had_smem);
  const uint32_t off0 = (uint32_t)(k0 * RS + 128 * u) * 2, off1 = (uint32_t)(k1 * RS + 128 * u) * 2;

  auto fetch = [&](int64_t row, int region) {
    const T* xr = x + row * ldx;
    T* dst = reinterpret_cast<T*>(had_smem + (size_t)region * region_bytes);
    for (int ch = tid; ch < base * (P / 8); ch += NTHREADS) {
      const int a = ch >> (LOGP - 3), cb = ch & (P / 8 - 1);
      had_cp_async16(dst + a * RS + cb * 8, xr + (size_t)a * P + cb * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int64_t row = blockIdx.x;
  int reg = 0;                                   // region of the current row
  if (row < rows) fetch(row, 0);
  for (; row < rows; row += gridDim.x) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                             // this row has landed; the previous row's second pass is over
    const int reg1 = reg + 1 >= 3 ? reg - 2 : reg + 1, reg2 = reg + 2 >= 3 ? reg - 1 : reg + 2;
    if (row + gridDim.x < rows) fetch(row + gridDim.x, reg2);
    const uint32_t raw_base = smem0 + (uint32_t)reg * region_bytes;

    float acc[16][4];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
      uint32_t b[6];
      if constexpr (KT == 1) {
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                     : "=r"(b[0]), "=r"(b[1]) : "r"(raw_base + off0 + t * 16));
      } else {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(raw_base + off0 + t * 16));
        if constexpr (KT == 3)
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                       : "=r"(b[4]), "=r"(b[5]) : "r"(raw_base + off1 + t * 16));
      }
#pragma unroll
      for (int kt = 0; kt < KT; ++kt) MmaOp<T>::mma(acc[t], afrag[kt], b[2 * kt], b[2 * kt + 1]);
    }
    // b = 128 u + 8 t + 2 c + e: bit 0 is the accumulator pair, bits 3..6 the n-tile index
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float a0 = acc[t][0], a1 = acc[t][1], a2 = acc[t][2], a3 = acc[t][3];
      acc[t][0] = a0 + a1; acc[t][1] = a0 - a1; acc[t][2] = a2 + a3; acc[t][3] = a2 - a3;
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1)
#pragma unroll
      for (int t = 0; t < 16; ++t)
        if (!(t & s)) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = acc[t][j], hi = acc[t | s][j];
            acc[t][j] = lo + hi;
            acc[t | s][j] = lo - hi;
          }
        }
    __syncthreads();                     // every warp has read its part of the raw row: the space becomes the fp32 tile
    // fp32 tile: row a' in region reg (a' < base / 2) or reg1; inside a row the two 16-byte halves of every odd
    // 32-float block are swapped, so that the second pass reads 16-byte vectors without bank conflicts
    float* f_lo = reinterpret_cast<float*>(had_smem + (size_t)reg * region_bytes);
    float* f_hi = reinterpret_cast<float*>(had_smem + (size_t)reg1 * region_bytes) - (size_t)half_rows * RS;
    {
      const int ra = 16 * mt + g, rb = ra + 8;
      float* fa = (ra < half_rows ? f_lo : f_hi) + ra * RS + 128 * u;
      float* fb2 = (rb < half_rows ? f_lo : f_hi) + rb * RS + 128 * u;
      const int c_plain = 2 * c, c_swap = (2 * c) ^ 4;      // column inside the 8-float tile, halves swapped or not
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int col = 8 * t + ((t & 4) ? c_swap : c_plain);   // bit 5 of the column index set <=> t & 4
        if (ra < base) *reinterpret_cast<float2*>(fa + col) = make_float2(acc[t][0], acc[t][1]);
        if (rb < base) *reinterpret_cast<float2*>(fb2 + col) = make_float2(acc[t][2], acc[t][3]);
      }
    }
    __syncthreads();
    T* yr = y + row * ldy;
    for (int task = tid; task < base * 16; task += NTHREADS) {
      const int ap = task >> 4, q = task & 15;
      const int flip = (q >> 2) & 1;
      const float* src = (ap < half_rows ? f_lo : f_hi) + ap * RS + 8 * q;
      float v[NU][8];
#pragma unroll
      for (int h = 0; h < NU; ++h) {
        const float4 lo = *reinterpret_cast<const float4*>(src + 128 * h + 4 * flip);
        const float4 hi = *reinterpret_cast<const float4*>(src + 128 * h + 4 * (flip ^ 1));
        v[h][0] = lo.x; v[h][1] = lo.y; v[h][2] = lo.z; v[h][3] = lo.w;
        v[h][4] = hi.x; v[h][5] = hi.y; v[h][6] = hi.z; v[h][7] = hi.w;
      }
#pragma unroll
      for (int h = 0; h < NU; ++h)
#pragma unroll
        for (int s = 2; s < 8; s <<= 1)
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (!(e & s)) {
              const float lo = v[h][e], hi = v[h][e | s];
              v[h][e] = lo + hi;
              v[h][e | s] = lo - hi;
            }
#pragma unroll
      for (int s = 1; s < NU; s <<= 1)
#pragma unroll
        for (int h = 0; h < NU; ++h)
          if (!(h & s)) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float lo = v[h][e], hi = v[h | s][e];
              v[h][e] = lo + hi;
              v[h | s][e] = lo - hi;
            }
          }
#pragma unroll
      for (int h = 0; h < NU; ++h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[h][e] *= scale;
        Elem<T>::store8(yr + (size_t)ap * P + 128 * h + 8 * q, v[h]);
      }
    }
    reg = reg2;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(128) hadamard_split_kernel(const T* __restrict__ x, int64_t ldx,
                                                             T* __restrict__ y, int64_t ldy, int P, int B,
                                                             float scale, const HadSigns signs, int pdl_trigger) {
  __shared__ __align__(16) float buf[1024];
  // In a decode chain the linear behind this kernel starts its weight stream right away.  The kernel itself is a plain
  // stream-ordered launch: started as a programmatic dependent of its producer it gained 0.5 us per Llama layer and
  // lost 1 us per Mamba layer (its early-resident successor competes with the producer's own stream).
  if (pdl_trigger) pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31;
  const int seg = blockIdx.x;
  const T* xr = x + (int64_t)blockIdx.y * ldx;
  T* yr = y + (int64_t)blockIdx.y * ldy + (size_t)seg * P;
  const uint64_t mask = signs.row[seg];
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  // The B segment loads are independent; they are issued 16 at a time (raw 16-byte vectors for 16-bit types)
  // so that a row costs two memory round trips instead of one per segment.
  constexpr int kBatch = 16;
  for (int a0 = 0; a0 < B; a0 += kBatch) {
    if constexpr (sizeof(T) == 2) {
      uint4 raw[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
        if (a0 + i < B) raw[i] = *reinterpret_cast<const uint4*>(xr + (size_t)(a0 + i) * P + tid * 8);
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
        if (a0 + i < B) {
          float t[8];
          Elem<T>::unpack8(raw[i], t);
          const float sg = ((mask >> (a0 + i)) & 1ull) ? -1.f : 1.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = fmaf(sg, t[e], v[e]);
        }
    } else {
#pragma unroll 4
      for (int i = 0; i < kBatch; ++i)
        if (a0 + i < B) {
          float t[8];
          Elem<T>::load8(xr + (size_t)(a0 + i) * P + tid * 8, t);
          const float sg = ((mask >> (a0 + i)) & 1ull) ? -1.f : 1.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = fmaf(sg, t[e], v[e]);
        }
    }
  }
  butterflies<8>(v);
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    if ((8 << s) < P) {
      const bool upper = (lane >> s) & 1;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float o = __shfl_xor_sync(0xffffffffu, v[i], 1 << s);
        v[i] = upper ? (o - v[i]) : (v[i] + o);
      }
    }
  }
  if (P > 256) {
    float4* d = reinterpret_cast<float4*>(buf + tid * 8);
    d[0] = make_float4(v[0], v[1], v[2], v[3]);
    d[1] = make_float4(v[4], v[5], v[6], v[7]);
    __syncthreads();
    if (P == 512) strided_pass<2>(buf, P, 256, tid, blockDim.x);
    else strided_pass<4>(buf, P, 256, tid, blockDim.x);
    __syncthreads();
    const float4* s4 = reinterpret_cast<const float4*>(buf + tid * 8);
    const float4 a = s4[0], b = s4[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= scale;
  Elem<T>::store8(yr + tid * 8, v);
}

// The few-row kernel again, for a tensor-parallel layer: the fp16 rows are read from this rank's feature area, where
// the column shards of all ranks arrive as 8-byte words {2 halves, epoch} (stored there by the epilogue of the
// column-parallel launch before this one).  A word whose epoch is not this call's yet is read again (bounded; a wait
// that gives up raises UNIQL_STATUS_WAIT_TIMEOUT).  The epoch of the call is this rank's gather counter + 1; this
// kernel advances the counter when it ends, so launches of any width may share a communicator.
__global__ void __launch_bounds__(128) hadamard_split_feat_kernel(const unsigned char* area, size_t gather_off,
                                                                  size_t epoch_off, int64_t feat_cap, __half* __restrict__ y,
                                                                  int64_t ldy, int P, int B, float scale,
                                                                  const HadSigns signs, int* status_word) {
  __shared__ __align__(16) float buf[1024];
  pdl_launch_dependents();                       // the linear behind this kernel only prefetches until it waits on us
  const int tid = threadIdx.x, lane = tid & 31;
  const int seg = blockIdx.x, row = blockIdx.y;
  // the words of this call carry (this rank's gather counter + 1): the producer launches of all ranks tagged them so
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(area + epoch_off) + 1;
  const uint2* xr = reinterpret_cast<const uint2*>(area + gather_off) +
                    ((size_t)(epoch & 1u) * 16 + row) * (size_t)(feat_cap >> 1);
  __half* yr = y + (int64_t)row * ldy + (size_t)seg * P;
  const uint64_t mask = signs.row[seg];
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  bool failed = false;
  constexpr int kBatch = 8;
  for (int a0 = 0; a0 < B; a0 += kBatch) {
    uint4 w[kBatch][2];                          // 4 words = 8 halves per source segment
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (a0 + i < B) {
        const uint2* src = xr + (((size_t)(a0 + i) * P + tid * 8) >> 1);
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[i][0].x), "=r"(w[i][0].y), "=r"(w[i][0].z), "=r"(w[i][0].w) : "l"(src) : "memory");
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[i][1].x), "=r"(w[i][1].y), "=r"(w[i][1].z), "=r"(w[i][1].w) : "l"(src + 2) : "memory");
      }
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (a0 + i < B) {
        const uint2* src = xr + (((size_t)(a0 + i) * P + tid * 8) >> 1);
        int spin = 0;
        while ((w[i][0].y != epoch || w[i][0].w != epoch || w[i][1].y != epoch || w[i][1].w != epoch) && !failed) {
          if (++spin > (1 << 22)) { failed = true; break; }
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[i][0].x), "=r"(w[i][0].y), "=r"(w[i][0].z), "=r"(w[i][0].w) : "l"(src) : "memory");
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[i][1].x), "=r"(w[i][1].y), "=r"(w[i][1].z), "=r"(w[i][1].w) : "l"(src + 2) : "memory");
        }
        const uint4 raw = make_uint4(w[i][0].x, w[i][0].z, w[i][1].x, w[i][1].z);
        float t[8];
        Elem<__half>::unpack8(raw, t);
        const float sg = ((mask >> (a0 + i)) & 1ull) ? -1.f : 1.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = fmaf(sg, t[e], v[e]);
      }
  }
  if (failed && status_word) atomicOr(status_word, UNIQL_STATUS_WAIT_TIMEOUT);
  butterflies<8>(v);
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    if ((8 << s) < P) {
      const bool upper = (lane >> s) & 1;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float o = __shfl_xor_sync(0xffffffffu, v[i], 1 << s);
        v[i] = upper ? (o - v[i]) : (v[i] + o);
      }
    }
  }
  if (P > 256) {
    float4* d = reinterpret_cast<float4*>(buf + tid * 8);
    d[0] = make_float4(v[0], v[1], v[2], v[3]);
    d[1] = make_float4(v[4], v[5], v[6], v[7]);
    __syncthreads();
    if (P == 512) strided_pass<2>(buf, P, 256, tid, blockDim.x);
    else strided_pass<4>(buf, P, 256, tid, blockDim.x);
    __syncthreads();
    const float4* s4 = reinterpret_cast<const float4*>(buf + tid * 8);
    const float4 a = s4[0], b = s4[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= scale;
  Elem<__half>::store8(yr + tid * 8, v);
  // The last CTA of the launch to get here (ticket, no waiting) advances the gather counter: every CTA has read it and
  // every word of this call has been consumed; the next producer launch is ordered behind this kernel.
  __syncthreads();
  if (tid == 0) {
    unsigned int* ticket = reinterpret_cast<unsigned int*>(const_cast<unsigned char*>(area) + epoch_off + 4);
    const unsigned int total = gridDim.x * gridDim.y;
    if (atomicAdd(ticket, 1u) == total - 1) {
      *ticket = 0;
      *reinterpret_cast<volatile uint32_t*>(const_cast<unsigned char*>(area) + epoch_off) = epoch;
    }
  }
}

// Segment layout of the few-row kernels: dim = B segments of Ps points.  Returns false if the size does not fit them.
// The sign words of the last few sizes are remembered (a decode loop asks for the same one on every step).
static bool split_layout(int64_t dim, int base, int64_t* Ps_out, int64_t* B_out, HadSigns* signs) {
  const int64_t P = dim / base;
  if (P < 256) return false;
  int64_t Ps = P < 512 ? P : 512;
  int64_t Q = P / Ps;
  if (base * Q > 64) { Ps = 1024; Q = P / Ps; }
  const int64_t B = base * Q;
  if (!(B <= 64 && Ps <= 1024 && Q >= 1)) return false;
  *Ps_out = Ps;
  *B_out = B;
  struct Entry { int64_t dim; unsigned gen; HadSigns signs; };
  static std::mutex mu;
  static Entry cache[8];
  static int used = 0, next = 0;
  unsigned gen;
  {
    std::lock_guard<std::mutex> lk(g_base_mu);
    gen = g_base_generation;
  }
  {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < used; ++i)
      if (cache[i].dim == dim && cache[i].gen == gen) { *signs = cache[i].signs; return true; }
  }
  int8_t h[1600];
  if (base > 1) base_matrix(base, h);
  for (int i = 0; i < 64; ++i) signs->row[i] = 0;
  for (int s1 = 0; s1 < B; ++s1)
    for (int s2 = 0; s2 < B; ++s2) {
      const int a1 = (int)(s1 / Q), h1 = (int)(s1 % Q), a2 = (int)(s2 / Q), h2 = (int)(s2 % Q);
      int neg = (base > 1 && h[a1 * base + a2] < 0) ? 1 : 0;
      neg ^= __builtin_popcount((unsigned)(h1 & h2)) & 1;
      if (neg) signs->row[s1] |= (1ull << s2);
    }
  std::lock_guard<std::mutex> lk(mu);
  cache[next] = {dim, gen, *signs};
  next = (next + 1) % 8;
  if (used < 8) ++used;
  return true;
}

int launch_hadamard_feat(const CommView& cv, void* y, int64_t ldy, int64_t rows, int64_t dim, float scale,
                         int* status_word, cudaStream_t stream) {
  const int base = hadamard_base_of(dim);
  if (base == 0 || dim > cv.feat_cap || rows < 1 || rows > 16) return UNIQL_ESHAPE;
  HadSigns signs;
  int64_t Ps = 0, B = 0;
  if (!split_layout(dim, base, &Ps, &B, &signs)) return UNIQL_ESHAPE;
  dim3 grid((unsigned)B, (unsigned)rows);
  hadamard_split_feat_kernel<<<grid, (int)(Ps / 8), 0, stream>>>(cv.bufs[cv.rank], cv.gather_off, cv.gather_epoch_off,
                                                               cv.feat_cap, (__half*)y, ldy, (int)Ps, (int)B, scale,
                                                               signs, status_word);
  return launch_status();
}

int launch_hadamard(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t dim, float scale,
                    int dtype, bool pdl_trigger, cudaStream_t stream) {
  const int base = hadamard_base_of(dim);
  if (base == 0) return UNIQL_ESHAPE;
  const int64_t P = dim / base;
  if (P < 8 || dim > 40960) return UNIQL_ESHAPE;
  if (rows == 0) return UNIQL_OK;
  int cur_dev = 0;
  cudaGetDevice(&cur_dev);
  if (cur_dev < 0 || cur_dev >= 64) cur_dev = 0;
  HadSigns signs;

  // ---- few rows: one CTA per (segment, row) ----
  if (rows <= 16 && P >= 256 && !(x == y)) {
    int64_t Ps = 0, B = 0;
    if (split_layout(dim, base, &Ps, &B, &signs)) {
      dim3 grid((unsigned)B, (unsigned)rows);
      const int threads = (int)(Ps / 8);
      const int trig = pdl_trigger ? 1 : 0;
      if (dtype == UNIQL_F16)
        hadamard_split_kernel<__half><<<grid, threads, 0, stream>>>((const __half*)x, ldx, (__half*)y, ldy, (int)Ps, (int)B, scale, signs, trig);
      else if (dtype == UNIQL_BF16)
        hadamard_split_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy, (int)Ps, (int)B, scale, signs, trig);
      else if (dtype == UNIQL_F32)
        hadamard_split_kernel<float><<<grid, threads, 0, stream>>>((const float*)x, ldx, (float*)y, ldy, (int)Ps, (int)B, scale, signs, trig);
      else return UNIQL_EDTYPE;
      return launch_status();
    }
  }
  for (int i = 0; i < 64; ++i) signs.row[i] = 0;
  int8_t h[1600];
  if (base > 1) base_matrix(base, h);

  // ---- many rows of a 16-bit type, 128 <= P <= 512: base matrix on the tensor cores ----
  if (dtype != UNIQL_F32) {
    int mbase = base;
    int64_t mP = P;
    if (base == 1) {                       // power of two: H_16 or H_32 (Sylvester) takes the base matrix's place
      mbase = dim >= 16384 ? 32 : 16;
      mP = dim / mbase;
    }
    if (mP == 128 || mP == 256 || mP == 512) {
      HadSigns ms;
      for (int i = 0; i < 64; ++i) ms.row[i] = 0;
      for (int i = 0; i < mbase; ++i)
        for (int j = 0; j < mbase; ++j) {
          const bool neg = base == 1 ? (__builtin_popcount((unsigned)(i & j)) & 1) : (h[i * base + j] < 0);
          if (neg) ms.row[i] |= (1ull << j);
        }
      const int MTv = (mbase + 15) / 16, logp = mP == 128 ? 7 : mP == 256 ? 8 : 9;
      const size_t smem = (size_t)3 * mbase * (size_t)(mP + 8) * 2;      // three raw-row regions
      const int threads = MTv * (int)(mP / 128) * 32;
#define UNIQL_HAD_MMA_CASE(T, MT_, LP_)                                                                       \
  do {                                                                                                        \
    static thread_local int ctas_per_sm[64] = {};  /* function attributes and occupancy are per device */     \
    if (!ctas_per_sm[cur_dev]) {                                                                              \
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(hadamard_mma_kernel<T, MT_, LP_>,                                   \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,                        \
                                          (int)(3 * 16 * MT_ * ((1 << LP_) + 8) * 2)));                       \
      int occ = 0;                                                                                            \
      UNIQL_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(                                           \
          &occ, hadamard_mma_kernel<T, MT_, LP_>, threads, (size_t)(3 * 16 * MT_ * ((1 << LP_) + 8) * 2)));   \
      ctas_per_sm[cur_dev] = occ < 1 ? 1 : (occ > 4 ? 4 : occ);                                               \
    }                                                                                                         \
    const int64_t max_ctas = (int64_t)ctas_per_sm[cur_dev] * device_info().sm_count;                          \
    const unsigned grid = (unsigned)(rows < max_ctas ? rows : max_ctas);                                      \
    hadamard_mma_kernel<T, MT_, LP_><<<grid, threads, smem, stream>>>((const T*)x, ldx, (T*)y, ldy, rows, mbase, \
                                                                      scale, ms, pdl_trigger ? 1 : 0);        \
    return launch_status();                                                                                   \
  } while (0)
#define UNIQL_HAD_MMA_LOGP(T, MT_)                                                                            \
  do {                                                                                                        \
    if (logp == 7) UNIQL_HAD_MMA_CASE(T, MT_, 7);                                                             \
    else if (logp == 8) UNIQL_HAD_MMA_CASE(T, MT_, 8);                                                        \
    else UNIQL_HAD_MMA_CASE(T, MT_, 9);                                                                       \
  } while (0)
#define UNIQL_HAD_MMA_MT(T)                                                                                   \
  do {                                                                                                        \
    if (MTv == 1) UNIQL_HAD_MMA_LOGP(T, 1);                                                                   \
    else if (MTv == 2) UNIQL_HAD_MMA_LOGP(T, 2);                                                              \
    else UNIQL_HAD_MMA_LOGP(T, 3);                                                                            \
  } while (0)
      if (dtype == UNIQL_F16) UNIQL_HAD_MMA_MT(__half);
      else if (dtype == UNIQL_BF16) UNIQL_HAD_MMA_MT(__nv_bfloat16);
      else return UNIQL_EDTYPE;
#undef UNIQL_HAD_MMA_MT
#undef UNIQL_HAD_MMA_LOGP
#undef UNIQL_HAD_MMA_CASE
    }
  }

  // ---- a base matrix replaced at run time: the kernels below have the built-in signs compiled in ----
  if (base > 1 && base_is_custom(base)) {
    for (int i = 0; i < base; ++i)
      for (int j = 0; j < base; ++j)
        if (h[i * base + j] < 0) signs.row[i] |= (1ull << j);
    const size_t smem = (size_t)dim * sizeof(float);
#define UNIQL_HAD_RT_LAUNCH(T)                                                                                \
  do {                                                                                                        \
    static thread_local bool attr_done[64] = {};   /* function attributes are per device */                   \
    if (!attr_done[cur_dev]) {                                                                                \
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(hadamard_rt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                          40960 * (int)sizeof(float)));                                       \
      attr_done[cur_dev] = true;                                                                              \
    }                                                                                                         \
    for (int64_t r0 = 0; r0 < rows; r0 += (int64_t)1 << 30) {                                                 \
      const int64_t nr = rows - r0 < ((int64_t)1 << 30) ? rows - r0 : ((int64_t)1 << 30);                     \
      hadamard_rt_kernel<T><<<(unsigned)nr, 256, smem, stream>>>((const T*)x + r0 * ldx, ldx, (T*)y + r0 * ldy, ldy, \
                                                                 (int)dim, (int)P, base, scale, signs,        \
                                                                 pdl_trigger ? 1 : 0);                        \
    }                                                                                                         \
  } while (0)
    if (dtype == UNIQL_F16) UNIQL_HAD_RT_LAUNCH(__half);
    else if (dtype == UNIQL_BF16) UNIQL_HAD_RT_LAUNCH(__nv_bfloat16);
    else if (dtype == UNIQL_F32) UNIQL_HAD_RT_LAUNCH(float);
    else return UNIQL_EDTYPE;
#undef UNIQL_HAD_RT_LAUNCH
    return launch_status();
  }

  // ---- many rows, P >= 32 and more stages than fit the register + shuffle pass: 32 elements per thread ----
  if (P >= 32 && !(base == 1 && P <= 256)) {
    int threads = (int)((dim / 32 + 31) / 32 * 32);
    if (threads < 64) threads = 64;
    const int max_threads = dim > 8192 ? 256 : 128;
    if (threads > max_threads) threads = max_threads;
    const size_t smem = (size_t)(dim + dim / 8) * sizeof(float);
#define UNIQL_HAD32_LAUNCH(T)                                                                                 \
  do {                                                                                                        \
    static thread_local bool attr_done[64] = {};   /* function attributes are per device */                   \
    if (smem > 48 * 1024 && !attr_done[cur_dev]) {                                                            \
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(hadamard_rows32_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                          (40960 + 40960 / 8) * (int)sizeof(float)));                         \
      attr_done[cur_dev] = true;                                                                              \
    }                                                                                                         \
    for (int64_t r0 = 0; r0 < rows; r0 += (int64_t)1 << 30) {                                                 \
      const int64_t nr = rows - r0 < ((int64_t)1 << 30) ? rows - r0 : ((int64_t)1 << 30);                     \
      hadamard_rows32_kernel<T><<<(unsigned)nr, threads, smem, stream>>>(                                     \
          (const T*)x + r0 * ldx, ldx, (T*)y + r0 * ldy, ldy, (int)dim, (int)P, base, scale, pdl_trigger ? 1 : 0); \
    }                                                                                                         \
  } while (0)
    if (dtype == UNIQL_F16) UNIQL_HAD32_LAUNCH(__half);
    else if (dtype == UNIQL_BF16) UNIQL_HAD32_LAUNCH(__nv_bfloat16);
    else if (dtype == UNIQL_F32) UNIQL_HAD32_LAUNCH(float);
    else return UNIQL_EDTYPE;
#undef UNIQL_HAD32_LAUNCH
    return launch_status();
  }

  // Small CTAs: many independent CTAs per SM in different phases (load, butterflies, store) overlap better than a few
  // large ones.  128 threads up to 8192 elements per row, 256 beyond (measured on B200: 14336 -> 689 us for 16384 rows
  // with 256 threads, 773 with 512, 870 with 128; 4096 -> 163 / 202 / 220 us with 128 / 256 / 512).  Very short rows
  // share a CTA so that every thread still has a chunk.
  int rpc = (int)((1024 + dim - 1) / dim);
  if (rpc < 1) rpc = 1;
  if (rpc > 8) rpc = 8;
  const int64_t want_ctas = 4 * (int64_t)device_info().sm_count;
  while (rpc > 1 && (rows + rpc - 1) / rpc < want_ctas) --rpc;
  int threads = (int)(((int64_t)rpc * dim / 8 + 31) / 32 * 32);
  if (threads < 64) threads = 64;
  const int max_threads = dim > 8192 ? 256 : 128;
  if (threads > max_threads) threads = max_threads;
  const size_t smem = (size_t)rpc * dim * sizeof(float);

#define UNIQL_HAD_LAUNCH(T)                                                                                   \
  do {                                                                                                        \
    static thread_local bool attr_done[64] = {};   /* function attributes are per device */                   \
    if (smem > 48 * 1024 && !attr_done[cur_dev]) {                                                            \
      UNIQL_CUDA_TRY(cudaFuncSetAttribute(hadamard_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                          40960 * (int)sizeof(float)));                                       \
      attr_done[cur_dev] = true;                                                                              \
    }                                                                                                         \
    const int64_t step = ((int64_t)1 << 30) * rpc;                                                            \
    for (int64_t r0 = 0; r0 < rows; r0 += step) {                                                             \
      const int64_t nr = rows - r0 < step ? rows - r0 : step;                                                 \
      hadamard_kernel<T><<<(unsigned)((nr + rpc - 1) / rpc), threads, smem, stream>>>(                        \
          (const T*)x + r0 * ldx, ldx, (T*)y + r0 * ldy, ldy, nr, rpc, (int)dim, (int)P, base, scale,         \
          pdl_trigger ? 1 : 0);                                                                               \
    }                                                                                                         \
  } while (0)

  if (dtype == UNIQL_F16) UNIQL_HAD_LAUNCH(__half);
  else if (dtype == UNIQL_BF16) UNIQL_HAD_LAUNCH(__nv_bfloat16);
  else if (dtype == UNIQL_F32) UNIQL_HAD_LAUNCH(float);
  else return UNIQL_EDTYPE;
#undef UNIQL_HAD_LAUNCH
  return launch_status();
}

}  // namespace uniql

extern "C" int uniql_hadamard(const void* x, void* y, int64_t rows, int64_t dim, float scale, int dtype,
                              void* stream) {
  using namespace uniql;
  if (rows < 0 || dim <= 0) return UNIQL_EINVAL;
  if (dtype != UNIQL_F16 && dtype != UNIQL_BF16 && dtype != UNIQL_F32) return UNIQL_EDTYPE;
  if (hadamard_base_of(dim) == 0) return UNIQL_ESHAPE;
  if (rows == 0) return UNIQL_OK;
  if (!x || !y || !aligned16(x) || !aligned16(y)) return UNIQL_EINVAL;
  return launch_hadamard(x, dim, y, dim, rows, dim, scale, dtype, false, (cudaStream_t)stream);
}

extern "C" int uniql_hadamard_set_base_matrix(int base, const int8_t* h) { return uniql::set_base_matrix(base, h); }

extern "C" int uniql_hadamard_base_matrix(int base, int8_t* out) {
  if (!out) return UNIQL_EINVAL;
  return uniql::base_matrix(base, out);
}
