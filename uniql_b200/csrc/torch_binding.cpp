// Torch-facing binding of the C ABI, the counterpart of UniQL's csrc/linear/quant_linear.cpp:6-25 (which binds
// w4a16o16_gemm with pybind) and csrc/embedding/quant_embedding.cpp.  The drop-in modules call these functions from
// their forward: shape checks, output allocation, scratch and the C-ABI call cost a few microseconds here instead of the
// tens of microseconds the same steps cost in Python over ctypes.  Nothing is computed in this file; every function ends
// in a call of libuniql_b200.so with raw pointers and the current stream.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <mutex>
#include <optional>
#include <unordered_map>
#include <vector>

#include "uniql_b200.h"

namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
  at::Tensor status;                                          // int32[1]
  std::unordered_map<uintptr_t, at::Tensor> scratch;          // per stream; counter region stays zero between launches
};

std::mutex g_mu;
DeviceState g_state[kMaxDevices];

at::Tensor status_tensor(int64_t device) {
  TORCH_CHECK(device >= 0 && device < kMaxDevices, "device index out of range");
  std::lock_guard<std::mutex> lk(g_mu);
  auto& st = g_state[device];
  if (!st.status.defined())
    st.status = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::Device(at::kCUDA, (c10::DeviceIndex)device)));
  return st.status;
}

// The caller holds a device guard for `device`.
at::Tensor scratch_for(int device, cudaStream_t stream, size_t need) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto& slot = g_state[device].scratch[(uintptr_t)stream];
  if (!slot.defined() || (size_t)slot.numel() < need) {
    size_t size = need < ((size_t)1 << 20) ? ((size_t)1 << 20) : need;
    size = (size + ((size_t)1 << 20) - 1) >> 20 << 20;
    slot = at::zeros({(int64_t)size}, at::TensorOptions().dtype(at::kByte).device(at::Device(at::kCUDA, (c10::DeviceIndex)device)));
  }
  return slot;
}

// Scratch requirement of the last few shapes (a decode loop repeats a handful of them).
struct NeedKey {
  int64_t v[8];
  bool operator==(const NeedKey& o) const {
    for (int i = 0; i < 8; ++i)
      if (v[i] != o.v[i]) return false;
    return true;
  }
};
template <typename F>
size_t cached_need(const NeedKey& key, F&& compute) {
  static thread_local std::vector<std::pair<NeedKey, size_t>> cache;
  for (const auto& e : cache)
    if (e.first == key) return e.second;
  const size_t need = compute();
  if (cache.size() >= 64) cache.clear();
  cache.emplace_back(key, need);
  return need;
}

void check_code(int code, const char* what) {
  if (code == UNIQL_OK) return;
  if (code == UNIQL_ECUDA)
    TORCH_CHECK(false, what, " failed: ", uniql_strerror(code), " (cudaError ", uniql_last_cuda_error(), ")");
  TORCH_CHECK(false, what, " failed: ", uniql_strerror(code));
}

void check_layer(const at::Tensor& weight, const at::Tensor& scale, const std::optional<at::Tensor>& bias,
                 int64_t n_out, int64_t* k_out, int64_t* n_store) {
  TORCH_CHECK(weight.is_cuda() && scale.is_cuda(), "weight and scale must be CUDA tensors (uniql_b200 has no CPU path)");
  TORCH_CHECK(weight.scalar_type() == at::kInt && scale.scalar_type() == at::kHalf, "weight must be int32 and scale float16");
  TORCH_CHECK(weight.dim() == 2 && scale.dim() == 2 && weight.is_contiguous() && scale.is_contiguous(),
              "weight and scale must be contiguous 2-D tensors");
  const int64_t k = weight.size(0) * 16, n = weight.size(1) / 2;
  TORCH_CHECK(scale.size(1) == n, "scale width does not match the packed weight");
  TORCH_CHECK(scale.size(0) * 128 == k, "only group size 128 is supported");
  TORCH_CHECK(n_out >= 1 && n_out <= n, "out_features exceeds the packed width");
  if (bias.has_value() && bias->defined())
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kHalf && bias->numel() >= n_out && bias->is_contiguous(),
                "bias must be a contiguous float16 CUDA tensor with at least out_features elements");
  *k_out = k;
  *n_store = n;
}

// x [..., in_features] -> fp16 [rows, k] with unit column stride, 16-byte aligned rows
at::Tensor rows_of(const at::Tensor& x, int64_t pad_in, int64_t k) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kHalf && x.dim() >= 1, "x must be a float16 CUDA tensor");
  at::Tensor x2 = x.dim() == 2 ? x : x.reshape({-1, x.size(-1)});
  if (pad_in > 0) x2 = at::constant_pad_nd(x2, {0, pad_in}, 0);
  TORCH_CHECK(x2.size(1) == k, "size_k mismatch: x has ", x2.size(1), " columns, packed weight covers ", k);
  if (x2.stride(1) != 1 || (x2.size(0) > 1 && x2.stride(0) % 8 != 0) || ((uintptr_t)x2.data_ptr()) % 16 != 0)
    x2 = x2.clone(at::MemoryFormat::Contiguous);
  return x2;
}

std::vector<int64_t> out_shape(const at::Tensor& x, int64_t n_out) {
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  shape.back() = n_out;
  return shape;
}

// W4A16B16O16Linear.forward (quantize/quant_linear_layers.py:91-116): y = x W^T (+ bias), padded input columns added
// here, padded output columns and the bias handled by the kernel epilogue; `hadamard` applies the online transform of
// size k to the rows first (the Hadamard module in front of down_proj / out_proj).
at::Tensor linear(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& scale,
                  const std::optional<at::Tensor>& bias, int64_t n_out, int64_t pad_in, bool hadamard) {
  int64_t k = 0, n = 0;
  check_layer(weight, scale, bias, n_out, &k, &n);
  const at::Tensor x2 = rows_of(x, pad_in, k);
  const int64_t m = x2.size(0);
  const c10::cuda::CUDAGuard guard(x2.device());
  const int dev = x2.device().index();
  at::Tensor out = at::empty(out_shape(x, n_out), x2.options());
  if (m == 0) return out;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int64_t had = hadamard ? k : 0;
  const size_t need = cached_need(NeedKey{{0, m, n, k, had, 0, 0, 0}}, [&] { return uniql_w4a16_scratch_bytes(m, n, k, had); });
  at::Tensor scratch = scratch_for(dev, stream, need);
  at::Tensor status = status_tensor(dev);
  const void* bias_ptr = (bias.has_value() && bias->defined()) ? bias->data_ptr() : nullptr;
  const int code = uniql_w4a16_linear(x2.data_ptr(), m > 1 ? x2.stride(0) : k, weight.data_ptr(), scale.data_ptr(), bias_ptr,
                                      out.data_ptr(), n_out, m, n, n_out, k, 128, had, scratch.data_ptr(),
                                      (size_t)scratch.numel(), (int*)status.data_ptr(), stream);
  check_code(code, "uniql_w4a16_linear");
  return out;
}

// One decode launch for projections that read the same activations (uniql_w4a16_linear_group): q/k/v, gate+up with
// act_fn(gate) * up (modeling/llama/llama_qblocks.py:48-51, :104-106), or one projection with the block's residual.
// Returns one tensor per projection (one tensor for the SwiGLU epilogue).  Up to 16 rows; 17..128 rows for plain
// outputs (one launch of the operand-swapped tensor-core kernel over all projections).
std::vector<at::Tensor> linear_group(const at::Tensor& x, const std::vector<at::Tensor>& weights,
                                     const std::vector<at::Tensor>& scales,
                                     const std::vector<std::optional<at::Tensor>>& biases,
                                     const std::vector<int64_t>& n_outs, int64_t epilogue,
                                     const std::optional<at::Tensor>& residual, int64_t pad_in, bool hadamard) {
  const int np = (int)weights.size();
  TORCH_CHECK(np >= 1 && np <= UNIQL_MAX_PROJ, "one launch takes 1 to ", UNIQL_MAX_PROJ, " projections");
  TORCH_CHECK((int)scales.size() == np && (int)biases.size() == np && (int)n_outs.size() == np,
              "weights, scales, biases and out_features must have one entry per projection");
  TORCH_CHECK(epilogue == UNIQL_EPILOGUE_NONE || epilogue == UNIQL_EPILOGUE_SWIGLU, "unknown epilogue");
  int64_t k = 0, ns[UNIQL_MAX_PROJ];
  for (int i = 0; i < np; ++i) {
    int64_t ki = 0;
    check_layer(weights[i], scales[i], biases[i], n_outs[i], &ki, &ns[i]);
    TORCH_CHECK(i == 0 || ki == k, "projections of one launch must share in_features");
    k = ki;
  }
  const at::Tensor x2 = rows_of(x, pad_in, k);
  const int64_t m = x2.size(0);
  TORCH_CHECK(m >= 1 && m <= 128, "grouped launches take 1 to 128 rows");
  TORCH_CHECK(m <= 16 || (epilogue == UNIQL_EPILOGUE_NONE && !hadamard && !(residual.has_value() && residual->defined())),
              "above 16 rows a grouped launch has plain outputs only");
  const c10::cuda::CUDAGuard guard(x2.device());
  const int dev = x2.device().index();
  const int nout = epilogue == UNIQL_EPILOGUE_SWIGLU ? 1 : np;
  std::vector<at::Tensor> outs;
  outs.reserve(nout);
  for (int i = 0; i < nout; ++i) outs.push_back(at::empty(out_shape(x, n_outs[i]), x2.options()));
  uniql_w4a16_proj proj[UNIQL_MAX_PROJ];
  for (int i = 0; i < np; ++i) {
    const at::Tensor& d = outs[i < nout ? i : nout - 1];
    proj[i].B = weights[i].data_ptr();
    proj[i].s = scales[i].data_ptr();
    proj[i].bias = (biases[i].has_value() && biases[i]->defined()) ? biases[i]->data_ptr() : nullptr;
    proj[i].D = d.data_ptr();
    proj[i].ldd = n_outs[i < nout ? i : nout - 1];
    proj[i].n = ns[i];
    proj[i].n_out = n_outs[i];
  }
  const void* res_ptr = nullptr;
  int64_t ldr = 0;
  at::Tensor res2;
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_cuda() && residual->scalar_type() == at::kHalf, "residual must be a float16 CUDA tensor");
    res2 = residual->dim() == 2 ? *residual : residual->reshape({-1, residual->size(-1)});
    if (res2.stride(1) != 1) res2 = res2.contiguous();
    TORCH_CHECK(res2.size(0) == m && res2.size(1) == n_outs[0], "residual must have the shape of the output");
    res_ptr = res2.data_ptr();
    ldr = res2.stride(0);
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  const int64_t had = hadamard ? k : 0;
  const size_t need = cached_need(
      NeedKey{{1 + epilogue + 2 * (had != 0), m, k, ns[0], np > 1 ? ns[1] : 0, np > 2 ? ns[2] : 0, np > 3 ? ns[3] : 0, np}},
      [&] { return uniql_w4a16_group_scratch_bytes(m, k, ns, np, (int)epilogue, had); });
  at::Tensor scratch = scratch_for(dev, stream, need);
  at::Tensor status = status_tensor(dev);
  const int code = uniql_w4a16_linear_group(x2.data_ptr(), m > 1 ? x2.stride(0) : k, m, k, proj, np, (int)epilogue, res_ptr,
                                            ldr, had, nullptr, 0, scratch.data_ptr(), (size_t)scratch.numel(),
                                            (int*)status.data_ptr(), stream);
  check_code(code, "uniql_w4a16_linear_group");
  return outs;
}

// W4O16Embedding.forward (quantize/quant_embedding_layers.py:49-51).
at::Tensor embedding(const at::Tensor& ids, const at::Tensor& weight, const at::Tensor& scales) {
  TORCH_CHECK(ids.is_cuda() && weight.is_cuda() && scales.is_cuda(), "input, weight and scale must be CUDA tensors");
  TORCH_CHECK(weight.dim() == 2 && weight.scalar_type() == at::kInt, "weight must be a 2-D int32 tensor");
  TORCH_CHECK(scales.dim() == 1 && scales.scalar_type() == at::kHalf && scales.numel() == weight.size(0),
              "scale must be a 1-D float16 tensor with one entry per table row");
  TORCH_CHECK((ids.dim() == 1 || ids.dim() == 2) && ids.scalar_type() == at::kLong, "input must be a 1-D or 2-D int64 tensor");
  const at::Tensor ids_c = ids.contiguous(), w = weight.contiguous(), s = scales.contiguous();
  const int64_t vocab = w.size(0), dim = w.size(1) * 8;
  std::vector<int64_t> shape(ids.sizes().begin(), ids.sizes().end());
  shape.push_back(dim);
  const c10::cuda::CUDAGuard guard(ids.device());
  const int dev = ids.device().index();
  at::Tensor out = at::empty(shape, at::TensorOptions().dtype(at::kHalf).device(ids.device()));
  at::Tensor status = status_tensor(dev);
  const int code = uniql_w4_embedding((const int64_t*)ids_c.data_ptr(), ids_c.numel(), w.data_ptr(), s.data_ptr(), out.data_ptr(), vocab, dim,
                                      (int*)status.data_ptr(), at::cuda::getCurrentCUDAStream(dev).stream());
  check_code(code, "uniql_w4_embedding");
  return out;
}

// act_fn(gate) * up between the launches of an MLP at more than 16 rows (uniql_silu_mul): one pass, PyTorch's roundings.
at::Tensor silu_mul(const at::Tensor& gate, const at::Tensor& up) {
  TORCH_CHECK(gate.is_cuda() && up.is_cuda() && gate.scalar_type() == at::kHalf && up.scalar_type() == at::kHalf,
              "gate and up must be float16 CUDA tensors");
  TORCH_CHECK(gate.sizes() == up.sizes() && gate.dim() >= 1, "gate and up must have the same shape");
  const int64_t cols = gate.size(-1);
  at::Tensor g2 = gate.reshape({-1, cols}), u2 = up.reshape({-1, cols});
  if (g2.stride(1) != 1 || g2.stride(0) % 8 || ((uintptr_t)g2.data_ptr()) % 16) g2 = g2.contiguous();
  if (u2.stride(1) != 1 || u2.stride(0) % 8 || ((uintptr_t)u2.data_ptr()) % 16) u2 = u2.contiguous();
  const c10::cuda::CUDAGuard guard(gate.device());
  at::Tensor out = at::empty(gate.sizes(), gate.options());
  const int code = uniql_silu_mul(g2.data_ptr(), g2.stride(0), u2.data_ptr(), u2.stride(0), out.data_ptr(), cols, g2.size(0),
                                  cols, at::cuda::getCurrentCUDAStream(gate.device().index()).stream());
  check_code(code, "uniql_silu_mul");
  return out;
}

// Hadamard.forward / had_transform (quantize/hadamard_helpers.py:18-48): y = H x * scale along the last axis.
at::Tensor hadamard(const at::Tensor& x, double scale) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (uniql_b200 has no CPU path)");
  int dtype = 0;
  if (x.scalar_type() == at::kHalf) dtype = UNIQL_F16;
  else if (x.scalar_type() == at::kBFloat16) dtype = UNIQL_BF16;
  else if (x.scalar_type() == at::kFloat) dtype = UNIQL_F32;
  else TORCH_CHECK(false, "unsupported dtype");
  const at::Tensor xc = x.contiguous();
  const int64_t dim = xc.dim() ? xc.size(-1) : 0;
  const int64_t rows = dim ? xc.numel() / dim : 0;
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(xc);
  const int code = uniql_hadamard(xc.data_ptr(), y.data_ptr(), rows, dim, (float)scale, dtype,
                                  at::cuda::getCurrentCUDAStream(x.device().index()).stream());
  check_code(code, "uniql_hadamard");
  return y;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "uniql_b200: torch binding of the C ABI (libuniql_b200.so)";
  m.def("abi_version", []() { return uniql_abi_version(); });
  m.def("status_tensor", &status_tensor, "int32[1] diagnostics word of a device");
  m.def("linear", &linear, "W4A16 linear forward");
  m.def("linear_group", &linear_group, "grouped W4A16 decode launch");
  m.def("embedding", &embedding, "4-bit embedding gather");
  m.def("hadamard", &hadamard, "Hadamard transform along the last axis");
  m.def("silu_mul", &silu_mul, "silu(gate) * up in one pass");
}
