// C-ABI entry points of the W4A16 linear and their regime dispatch (persistent streaming kernel for m <= 16,
// tcgen05 tensor-core kernels above), the grouped decode launch and its tensor-parallel form.
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

static bool use_tc(int64_t m, int64_t n, int64_t k) { return m > 16 && gemm_tc_supported(m, n, k); }

// Scratch of the single-projection entry point: what the decode kernel needs, or (tensor-core route with a
// Hadamard in front) the transformed activations.
static size_t linear_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t hadamard_dim) {
  if (use_tc(m, n, k))
    return UNIQL_SCRATCH_COUNTER_BYTES + (hadamard_dim ? align_up((size_t)m * k * 2, 256) : 0) +
           align_up(gemm_tc_scratch_bytes(m, n, k), 256);
  // decode kernel, in slabs of 16 rows when m > 16 (shapes the tensor-core kernels do not take)
  size_t need = decode_scratch_bytes(m > 16 ? 16 : m, k, &n, 1, UNIQL_EPILOGUE_NONE, m > 16 ? 0 : hadamard_dim, 0);
  if (m > 16) {
    if (m % 16) {
      const size_t t = decode_scratch_bytes(m % 16, k, &n, 1, UNIQL_EPILOGUE_NONE, 0, 0);
      if (t > need) need = t;
    }
    if (hadamard_dim) need += align_up((size_t)m * k * 2, 256);
  }
  return need;
}

static int check_proj(const uniql_w4a16_proj& q, int64_t k) {
  if (q.n <= 0 || q.n_out <= 0 || q.n_out > q.n) return UNIQL_EINVAL;
  if (q.n % 64 != 0 || q.n > (int64_t)1 << 22 || k > (int64_t)1 << 22) return UNIQL_ESHAPE;
  if (q.ldd < q.n_out) return UNIQL_EINVAL;
  if (!q.B || !q.s || !q.D) return UNIQL_EINVAL;
  if (!aligned16(q.B) || !aligned16(q.s) || (reinterpret_cast<uintptr_t>(q.D) & 1u)) return UNIQL_EINVAL;
  if (q.bias && (reinterpret_cast<uintptr_t>(q.bias) & 1u)) return UNIQL_EINVAL;
  return UNIQL_OK;
}

static int group_launch(const CommView* cv, int64_t k_offset, const void* A, int64_t lda, int64_t m, int64_t k,
                        const uniql_w4a16_proj* proj, int nproj, int epilogue, const void* residual, int64_t ldr,
                        int64_t hadamard_dim, const uniql_prefetch* next, int nnext, void* scratch,
                        size_t scratch_bytes, int* status_word, cudaStream_t stream) {
  if (!proj || nproj < 1 || nproj > UNIQL_MAX_PROJ || m < 0 || k <= 0) return UNIQL_EINVAL;
  if (k % 128 != 0) return UNIQL_ESHAPE;
  if (m > 16) {
    // 17..128 rows: the projections share one launch of the operand-swapped tensor-core kernel (plain outputs only:
    // the elementwise epilogues, the transform and the tensor-parallel exchanges belong to the decode kernel)
    if (m > 128 || cv || epilogue != UNIQL_EPILOGUE_NONE || residual || hadamard_dim) return UNIQL_ESHAPE;
    if (lda < k || lda % 8 != 0 || !A || !aligned16(A)) return UNIQL_EINVAL;
    LinearArgs la[UNIQL_MAX_PROJ];
    void* ds[UNIQL_MAX_PROJ];
    int64_t widths[UNIQL_MAX_PROJ];
    for (int i = 0; i < nproj; ++i) {
      const int st = check_proj(proj[i], k);
      if (st != UNIQL_OK) return st;
      la[i].B = proj[i].B; la[i].s = proj[i].s; la[i].bias = proj[i].bias; la[i].ldd = proj[i].ldd;
      la[i].n = proj[i].n; la[i].n_out = proj[i].n_out; la[i].k = k; la[i].status_word = status_word;
      ds[i] = proj[i].D;
      widths[i] = proj[i].n;
    }
    if (!gemm_tc_group_supported(m, k, widths, nproj)) return UNIQL_ESHAPE;
    return launch_gemm_tc_group(la, ds, nproj, (const __half*)A, lda, m, stream);
  }
  if (epilogue != UNIQL_EPILOGUE_NONE && epilogue != UNIQL_EPILOGUE_SWIGLU) return UNIQL_EINVAL;
  if (epilogue == UNIQL_EPILOGUE_SWIGLU && (nproj != 2 || proj[0].n != proj[1].n || proj[0].n_out != proj[1].n_out))
    return UNIQL_EINVAL;
  for (int i = 0; i < nproj; ++i) {
    const int st = check_proj(proj[i], k);
    if (st != UNIQL_OK) return st;
  }
  const bool gather_in = cv && cv->gather_in;
  if (!gather_in) {
    if (lda < k || lda % 8 != 0) return UNIQL_EINVAL;
    if (m > 0 && (!A || !aligned16(A))) return UNIQL_EINVAL;
  }
  if (residual) {
    if (nproj != 1 && epilogue != UNIQL_EPILOGUE_SWIGLU) return UNIQL_EINVAL;
    if (ldr < proj[0].n_out || (reinterpret_cast<uintptr_t>(residual) & 1u)) return UNIQL_EINVAL;
  }
  if (hadamard_dim != 0) {
    if (hadamard_base_of(hadamard_dim) == 0 || hadamard_dim > 40960) return UNIQL_ESHAPE;
    if (!cv && (hadamard_dim != k || k_offset != 0)) return UNIQL_ESHAPE;
  }
  if (cv && cv->gather_out) {
    if (nproj != 1 && epilogue != UNIQL_EPILOGUE_SWIGLU) return UNIQL_EINVAL;
    if (proj[0].n_out % 2) return UNIQL_ESHAPE;
  }
  if (m == 0) return UNIQL_OK;
  DecodeArgs a{};
  a.A = A; a.lda = lda; a.m = m; a.k = k; a.nproj = nproj;
  for (int i = 0; i < nproj; ++i) {
    a.proj[i].B = proj[i].B; a.proj[i].s = proj[i].s; a.proj[i].bias = proj[i].bias; a.proj[i].D = proj[i].D;
    a.proj[i].ldd = proj[i].ldd; a.proj[i].n = proj[i].n; a.proj[i].n_out = proj[i].n_out;
  }
  a.epilogue = epilogue;
  a.residual = residual; a.ldr = ldr;
  a.hadamard_dim = hadamard_dim; a.k_offset = k_offset;
  a.scratch = scratch; a.scratch_bytes = scratch_bytes;
  a.status_word = status_word;
  a.comm = cv;
  a.nprefetch = 0;
  if (next)
    for (int i = 0; i < nnext && a.nprefetch < UNIQL_MAX_PREFETCH; ++i)
      if (next[i].ptr && next[i].bytes) {
        a.prefetch_ptr[a.nprefetch] = next[i].ptr;
        a.prefetch_bytes[a.nprefetch] = next[i].bytes;
        ++a.nprefetch;
      }
  return launch_decode(a, stream);
}

}  // namespace uniql

extern "C" size_t uniql_w4a16_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t hadamard_dim) {
  if (m <= 0 || n <= 0 || k <= 0 || n % 64 || k % 128) return UNIQL_SCRATCH_COUNTER_BYTES;
  return uniql::linear_scratch_bytes(m, n, k, hadamard_dim);
}

extern "C" size_t uniql_w4a16_group_scratch_bytes(int64_t m, int64_t k, const int64_t* n, int nproj, int epilogue,
                                                  int64_t hadamard_dim) {
  if (!n || m <= 0 || m > 16 || k <= 0 || k % 128 || nproj < 1 || nproj > UNIQL_MAX_PROJ) return UNIQL_SCRATCH_COUNTER_BYTES;
  // the tensor-parallel form may be called with any k_offset: the requirement does not depend on it by more than
  // one tile per block and chunk, which the figure below already covers (one extra chunk)
  size_t a = uniql::decode_scratch_bytes(m, k, n, nproj, epilogue, hadamard_dim, 0);
  if (hadamard_dim && hadamard_dim != k) {
    for (int64_t off = 128; off < 512 && off + k <= hadamard_dim; off += 128) {
      const size_t b = uniql::decode_scratch_bytes(m, k, n, nproj, epilogue, hadamard_dim, off);
      if (b > a) a = b;
    }
  }
  return a;
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
  if (!scratch || scratch_bytes < linear_scratch_bytes(m, n, k, hadamard_dim) ||
      (reinterpret_cast<uintptr_t>(scratch) & 255u))
    return UNIQL_ESCRATCH;

  uniql_w4a16_proj q;
  q.B = B; q.s = s; q.bias = bias; q.D = D; q.ldd = ldd; q.n = n; q.n_out = n_out;
  if (m <= 16)
    return group_launch(nullptr, 0, A, lda, m, k, &q, 1, UNIQL_EPILOGUE_NONE, nullptr, 0, hadamard_dim, nullptr, 0,
                        scratch, scratch_bytes, status_word, stream);

  // m > 16: Hadamard (if any) as its own kernel into scratch, then the tensor-core kernels
  const __half* Ain = (const __half*)A;
  size_t used = UNIQL_SCRATCH_COUNTER_BYTES;
  const bool tc = use_tc(m, n, k);
  if (hadamard_dim) {
    const size_t xh_bytes = align_up((size_t)m * k * 2, 256);
    // the decode slabs below keep their tiles in front; the transformed rows sit at the end of the buffer
    __half* xh = (__half*)((char*)scratch + (tc ? used : scratch_bytes / 256 * 256 - xh_bytes));
    int st = launch_hadamard(A, lda, xh, k, m, k, (float)(1.0 / sqrt((double)k)), UNIQL_F16, false, stream);
    if (st != UNIQL_OK) return st;
    Ain = xh;
    lda = k;
    used += xh_bytes;
  }
  if (tc) {
    LinearArgs a;
    a.B = B; a.s = s; a.bias = bias; a.ldd = ldd; a.n = n; a.n_out = n_out; a.k = k; a.status_word = status_word;
    return launch_gemm_tc(a, Ain, lda, (__half*)D, m, stream);
  }
  const size_t slab_bytes = scratch_bytes - (hadamard_dim ? align_up((size_t)m * k * 2, 256) : 0);
  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const int64_t mc = m - m0 < 16 ? m - m0 : 16;
    q.D = (__half*)D + m0 * ldd;
    int st = group_launch(nullptr, 0, Ain + m0 * lda, lda, mc, k, &q, 1, UNIQL_EPILOGUE_NONE, nullptr, 0, 0, nullptr, 0,
                          scratch, slab_bytes, status_word, stream);
    if (st != UNIQL_OK) return st;
  }
  return UNIQL_OK;
}

extern "C" int uniql_w4a16_linear_group(const void* A, int64_t lda, int64_t m, int64_t k,
                                        const uniql_w4a16_proj* proj, int nproj, int epilogue, const void* residual,
                                        int64_t ldr, int64_t hadamard_dim, const uniql_prefetch* next, int nnext,
                                        void* scratch, size_t scratch_bytes, int* status_word, void* stream) {
  return uniql::group_launch(nullptr, 0, A, lda, m, k, proj, nproj, epilogue, residual, ldr, hadamard_dim, next, nnext,
                             scratch, scratch_bytes, status_word, (cudaStream_t)stream);
}

extern "C" int uniql_w4a16_linear_group_tp(void* comm, int flags, int64_t col_offset, int64_t k_offset, const void* A,
                                           int64_t lda, int64_t m, int64_t k, const uniql_w4a16_proj* proj, int nproj,
                                           int epilogue, const void* residual, int64_t ldr, int64_t hadamard_dim,
                                           const uniql_prefetch* next, int nnext, void* scratch,
                                           size_t scratch_bytes, int* status_word, void* stream) {
  using namespace uniql;
  if (!comm || (flags & ~(UNIQL_TP_REDUCE | UNIQL_TP_GATHER_OUT | UNIQL_TP_GATHER_IN))) return UNIQL_EINVAL;
  if ((flags & UNIQL_TP_REDUCE) && (flags & UNIQL_TP_GATHER_OUT)) return UNIQL_EINVAL;
  if ((flags & UNIQL_TP_GATHER_IN) && !hadamard_dim) return UNIQL_EINVAL;
  if (col_offset < 0 || k_offset < 0) return UNIQL_EINVAL;
  CommView cv;
  int st = comm_view(comm, &cv);
  if (st != UNIQL_OK) return st;
  cv.reduce = (flags & UNIQL_TP_REDUCE) ? 1 : 0;
  cv.gather_out = (flags & UNIQL_TP_GATHER_OUT) ? 1 : 0;
  cv.gather_in = (flags & UNIQL_TP_GATHER_IN) ? 1 : 0;
  cv.col_offset = col_offset;
  return group_launch(&cv, k_offset, A, lda, m, k, proj, nproj, epilogue, residual, ldr, hadamard_dim, next, nnext,
                      scratch, scratch_bytes, status_word, (cudaStream_t)stream);
}

extern "C" int uniql_w4a16_linear_allreduce(void* comm, const void* A, int64_t lda, const void* B, const void* s,
                                            const void* bias, void* D, int64_t ldd, int64_t m, int64_t n,
                                            int64_t n_out, int64_t k, int groupsize, void* scratch,
                                            size_t scratch_bytes, int* status_word, void* stream) {
  if (groupsize != 128) return groupsize == -1 ? UNIQL_EGROUPSIZE : UNIQL_EINVAL;
  if (n_out <= 0 || n_out > n) return UNIQL_EINVAL;
  uniql_w4a16_proj q;
  q.B = B; q.s = s; q.bias = bias; q.D = D; q.ldd = ldd; q.n = n; q.n_out = n_out;
  return uniql_w4a16_linear_group_tp(comm, UNIQL_TP_REDUCE, 0, 0, A, lda, m, k, &q, 1, UNIQL_EPILOGUE_NONE, nullptr, 0,
                                     0, nullptr, 0, scratch, scratch_bytes, status_word, stream);
}

extern "C" int uniql_abi_version(void) { return UNIQL_ABI_VERSION; }

extern "C" int uniql_last_cuda_error(void) { return uniql::g_last_cuda_error; }

extern "C" const char* uniql_strerror(int code) {
  switch (code) {
    case UNIQL_OK: return "ok";
    case UNIQL_EINVAL: return "invalid argument (null/misaligned pointer or bad size)";
    case UNIQL_EGROUPSIZE: return "unsupported groupsize: only group-128 scales are implemented (per-channel -1 is rejected)";
    case UNIQL_ESHAPE: return "unsupported shape (n % 64, k % 128, m > 16 for a decode-only entry point, Hadamard size, or communicator capacity)";
    case UNIQL_ESCRATCH: return "scratch buffer missing, misaligned or too small";
    case UNIQL_ECUDA: return "CUDA runtime error (see uniql_last_cuda_error)";
    case UNIQL_EDTYPE: return "unsupported element type";
    case UNIQL_ESTATIC: return "problem too large for the built-in scratch of uniql_w4a16_linear_static";
    default: return "unknown error";
  }
}
