// act_fn(gate) * up for batches the grouped decode launch does not cover (more than 16 rows): one pass over the two
// projection outputs instead of PyTorch's two (SiLU, then the product), with the roundings of the separate modules --
// fp16 SiLU, fp16 product (modeling/llama/llama_qblocks.py:48-51: down_proj(act_fn(gate_proj(x)) * up_proj(x))).
// HBM-bound: 6 bytes per element.
#include "common.cuh"

namespace uniql {

__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ gate, int64_t ldg,
                                                      const __half* __restrict__ up, int64_t ldu,
                                                      __half* __restrict__ out, int64_t ldo, int64_t rows,
                                                      int64_t cols8) {
  pdl_launch_dependents();
  pdl_wait();                                   // gate and up come from the launch right before this one
  const int64_t total = rows * cols8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols8, c = (i - r * cols8) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate + r * ldg + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(up + r * ldu + c);
    const __half2* gh = reinterpret_cast<const __half2*>(&g4);
    const __half2* uh = reinterpret_cast<const __half2*>(&u4);
    uint4 o4;
    __half2* oh = reinterpret_cast<__half2*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = __half22float2(gh[e]), uf = __half22float2(uh[e]);
      const __half2 act = __floats2half2_rn(gf.x / (1.0f + expf(-gf.x)), gf.y / (1.0f + expf(-gf.y)));
      const float2 af = __half22float2(act);
      oh[e] = __floats2half2_rn(af.x * uf.x, af.y * uf.y);
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o4;
  }
}

}  // namespace uniql

extern "C" int uniql_silu_mul(const void* gate, int64_t ldg, const void* up, int64_t ldu, void* out, int64_t ldo,
                              int64_t rows, int64_t cols, void* stream) {
  using namespace uniql;
  if (rows < 0 || cols < 0) return UNIQL_EINVAL;
  if (rows == 0 || cols == 0) return UNIQL_OK;
  if (!gate || !up || !out || !aligned16(gate) || !aligned16(up) || !aligned16(out)) return UNIQL_EINVAL;
  if (cols % 8 || ldg % 8 || ldu % 8 || ldo % 8 || ldg < cols || ldu < cols || ldo < cols) return UNIQL_ESHAPE;
  const int64_t total = rows * (cols / 8);
  int64_t ctas = (total + 255) / 256;
  const int64_t cap = 8 * (int64_t)device_info().sm_count;
  if (ctas > cap) ctas = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  UNIQL_CUDA_TRY(cudaLaunchKernelEx(&cfg, silu_mul_kernel, (const __half*)gate, ldg, (const __half*)up, ldu, (__half*)out,
                                    ldo, rows, cols / 8));
  return UNIQL_OK;
}
