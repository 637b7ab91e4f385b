// C-ABI entry point of the W4A16 linear and its regime dispatch (decode streaming kernel for m <= 16,
// tcgen05 tensor-core kernel above), plus the optional Hadamard prologue.
#include "common.cuh"
#include "linear_internal.cuh"

namespace uniql {

thread_local int g_last_cuda_error = 0;

const DeviceInfo& device_info() {
  static thread_local DeviceInfo info[64];
  static thread_local bool have[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!have[dev]) {
    int sms = 148, smem = 227 * 1024;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (sms <= 0) sms = 148;
    info[dev].sm_count = sms;
    info[dev].max_smem_optin = smem;
    have[dev] = true;
  }
  return info[dev];
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ScratchLayout {
  size_t xh_off, xh_bytes;        // Hadamard-transformed activations, fp16 [m, k]
  size_t part_off, part_bytes;    // split-k partials (decode) or tensor-core scratch
  size_t total;
};

static ScratchLayout scratch_layout(int64_t m, int64_t n, int64_t k, int64_t hadamard_dim) {
  ScratchLayout L;
  L.xh_off = UNIQL_SCRATCH_COUNTER_BYTES;
  L.xh_bytes = hadamard_dim ? align_up((size_t)m * k * 2, 256) : 0;
  L.part_off = L.xh_off + L.xh_bytes;
  size_t pb = 0;
  if (m > 16 && gemm_tc_supported(m, n, k)) {
    pb = gemm_tc_scratch_bytes(m, n, k);
  } else {
    // decode kernel, in slabs of 16 rows when m > 16
    pb = plan_gemv(m > 16 ? 16 : m, n, k).partial_bytes;
    if (m > 16 && m % 16) {
      size_t t = plan_gemv(m % 16, n, k).partial_bytes;
      if (t > pb) pb = t;
    }
  }
  L.part_bytes = align_up(pb, 256);
  L.total = L.part_off + L.part_bytes;
  return L;
}

}  // namespace uniql

extern "C" size_t uniql_w4a16_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t hadamard_dim) {
  if (m <= 0 || n <= 0 || k <= 0 || n % 64 || k % 128) return UNIQL_SCRATCH_COUNTER_BYTES;
  return uniql::scratch_layout(m, n, k, hadamard_dim).total;
}

extern "C" int uniql_w4a16_linear(const void* A, int64_t lda, const void* B, const void* s, const void* bias,
                                  void* D, int64_t ldd, int64_t m, int64_t n, int64_t n_out, int64_t k,
                                  int groupsize, int64_t hadamard_dim, void* scratch, size_t scratch_bytes,
                                  int* status_word, void* stream_) {
  using namespace uniql;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (groupsize != 128) return groupsize == -1 ? UNIQL_EGROUPSIZE : UNIQL_EINVAL;
  if (m < 0 || n <= 0 || k <= 0 || n_out <= 0 || n_out > n) return UNIQL_EINVAL;
  if (n % 64 != 0 || k % 128 != 0 || n > (int64_t)1 << 22 || k > (int64_t)1 << 22) return UNIQL_ESHAPE;
  if (lda < k || ldd < n_out || lda % 8 != 0) return UNIQL_EINVAL;
  if (hadamard_dim != 0 && (hadamard_dim != k || hadamard_base_of(k) == 0 || k > 40960)) return UNIQL_ESHAPE;
  if (m == 0) return UNIQL_OK;
  if (!A || !B || !s || !D) return UNIQL_EINVAL;
  if (!aligned16(A) || !aligned16(B) || !aligned16(s) || (reinterpret_cast<uintptr_t>(D) & 1u)) return UNIQL_EINVAL;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 1u)) return UNIQL_EINVAL;

  const ScratchLayout L = scratch_layout(m, n, k, hadamard_dim);
  if (!scratch || scratch_bytes < L.total || (reinterpret_cast<uintptr_t>(scratch) & 255u)) return UNIQL_ESCRATCH;

  LinearArgs a;
  a.B = B; a.s = s; a.bias = bias; a.ldd = ldd; a.n = n; a.n_out = n_out; a.k = k;
  a.counters = (int*)scratch;
  a.partials = (float*)((char*)scratch + L.part_off);
  a.partial_bytes = L.part_bytes;
  a.status_word = status_word;
  a.ar = nullptr;

  const __half* Ain = (const __half*)A;
  const bool decode = !(m > 16 && gemm_tc_supported(m, n, k));
  bool pdl = false;
  if (hadamard_dim) {
    __half* xh = (__half*)((char*)scratch + L.xh_off);
    pdl = decode;   // let the weight stream start while the transform runs
    int st = launch_hadamard(A, lda, xh, k, m, k, (float)(1.0 / sqrt((double)k)), UNIQL_F16, pdl, stream);
    if (st != UNIQL_OK) return st;
    Ain = xh;
    lda = k;
  }

  if (!decode) return launch_gemm_tc(a, Ain, lda, (__half*)D, m, stream);

  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const int64_t mc = m - m0 < 16 ? m - m0 : 16;
    const GemvPlan plan = plan_gemv(mc, n, k);
    int st = launch_gemv(a, Ain + m0 * lda, lda, (__half*)D + m0 * ldd, mc, plan, pdl && m0 == 0, stream);
    if (st != UNIQL_OK) return st;
  }
  return UNIQL_OK;
}

extern "C" int uniql_w4a16_linear_allreduce(void* comm, const void* A, int64_t lda, const void* B, const void* s,
                                            const void* bias, void* D, int64_t ldd, int64_t m, int64_t n,
                                            int64_t n_out, int64_t k, int groupsize, void* scratch,
                                            size_t scratch_bytes, int* status_word, void* stream_) {
  using namespace uniql;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (groupsize != 128) return groupsize == -1 ? UNIQL_EGROUPSIZE : UNIQL_EINVAL;
  if (!comm || m < 0 || n <= 0 || k <= 0 || n_out <= 0 || n_out > n) return UNIQL_EINVAL;
  if (m > 16) return UNIQL_ESHAPE;                       // decode sizes only: larger batches reduce separately
  if (n % 64 != 0 || k % 128 != 0 || n > (int64_t)1 << 22 || k > (int64_t)1 << 22) return UNIQL_ESHAPE;
  if (lda < k || ldd < n_out || lda % 8 != 0) return UNIQL_EINVAL;
  if (m == 0) return UNIQL_OK;
  if (!A || !B || !s || !D) return UNIQL_EINVAL;
  if (!aligned16(A) || !aligned16(B) || !aligned16(s) || (reinterpret_cast<uintptr_t>(D) & 1u)) return UNIQL_EINVAL;
  ArFuse ar;
  int st = comm_fuse_desc(comm, m, n, &ar);
  if (st != UNIQL_OK) return st;
  const ScratchLayout L = scratch_layout(m, n, k, 0);
  if (!scratch || scratch_bytes < L.total || (reinterpret_cast<uintptr_t>(scratch) & 255u)) return UNIQL_ESCRATCH;
  LinearArgs a;
  a.B = B; a.s = s; a.bias = bias; a.ldd = ldd; a.n = n; a.n_out = n_out; a.k = k;
  a.counters = (int*)scratch;
  a.partials = (float*)((char*)scratch + L.part_off);
  a.partial_bytes = L.part_bytes;
  a.status_word = status_word;
  a.ar = &ar;
  const GemvPlan plan = plan_gemv(m, n, k);
  return launch_gemv(a, (const __half*)A, lda, (__half*)D, m, plan, false, stream);
}

extern "C" int uniql_abi_version(void) { return UNIQL_ABI_VERSION; }

extern "C" int uniql_last_cuda_error(void) { return uniql::g_last_cuda_error; }

extern "C" const char* uniql_strerror(int code) {
  switch (code) {
    case UNIQL_OK: return "ok";
    case UNIQL_EINVAL: return "invalid argument (null/misaligned pointer or bad size)";
    case UNIQL_EGROUPSIZE: return "unsupported groupsize: only group-128 scales are implemented (per-channel -1 is rejected)";
    case UNIQL_ESHAPE: return "unsupported shape (n % 64, k % 128, or Hadamard size)";
    case UNIQL_ESCRATCH: return "scratch buffer missing, misaligned or too small";
    case UNIQL_ECUDA: return "CUDA runtime error (see uniql_last_cuda_error)";
    case UNIQL_EDTYPE: return "unsupported element type";
    case UNIQL_ESTATIC: return "problem too large for the built-in scratch of uniql_w4a16_linear_static";
    default: return "unknown error";
  }
}
