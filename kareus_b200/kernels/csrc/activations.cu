// GELU and GeGLU forward/backward (tanh approximation, the one Megatron's fused bias-GELU uses).
// The Llama/Qwen models of the benchmarks use SwiGLU (elementwise.cu); these cover the reference's
// other activation operators (kareus/megatron/core/extensions/ops/bias_gelu.py, bias_geglu.py).
#include <cuda_bf16.h>
#include "launch.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace kb {

__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * x * (1.f + 0.044715f * x * x)));
}
__device__ __forceinline__ float gelu_df(float x) {
  const float t = tanhf(0.7978845608028654f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.7978845608028654f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}

// mode 0: y = gelu(x) over n elements.  mode 1: x = [gate | up] rows of 2F, y = gelu(gate) * up.
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows, int F,
                                int gated) {
  const long total = rows * F;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / F;
    const int c = static_cast<int>(i % F);
    if (gated) {
      const float a = __bfloat162float(x[r * 2 * F + c]), b = __bfloat162float(x[r * 2 * F + F + c]);
      y[i] = __float2bfloat16(gelu_f(a) * b);
    } else {
      y[i] = __float2bfloat16(gelu_f(__bfloat162float(x[i])));
    }
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long rows, int F, int gated) {
  const long total = rows * F;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = __bfloat162float(dy[i]);
    if (gated) {
      const float a = __bfloat162float(x[r * 2 * F + c]), b = __bfloat162float(x[r * 2 * F + F + c]);
      dx[r * 2 * F + c] = __float2bfloat16(g * b * gelu_df(a));
      dx[r * 2 * F + F + c] = __float2bfloat16(g * gelu_f(a));
    } else {
      dx[i] = __float2bfloat16(g * gelu_df(__bfloat162float(x[i])));
    }
  }
}

}  // namespace kb

extern "C" int kb_gelu_fwd(const void* x, void* y, long rows, int F, int gated, cudaStream_t st) {
  long b = (rows * F + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  KB_LAUNCH(kb::gelu_fwd_kernel, (int)b, 256, 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, F, gated);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}
extern "C" int kb_gelu_bwd(const void* dy, const void* x, void* dx, long rows, int F, int gated, cudaStream_t st) {
  long b = (rows * F + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  KB_LAUNCH(kb::gelu_bwd_kernel, (int)b, 256, 0, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, rows,
                                              F, gated);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}
