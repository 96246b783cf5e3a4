// LayerNorm forward/backward and bias add / bias gradient for bf16 rows.
// The Llama and Qwen models of the benchmarks use RMSNorm without biases (elementwise.cu); these
// kernels cover the reference's LayerNorm option and bias-carrying linear layers
// (kareus/megatron/core/extensions/ops/te_norm.py, kareus/transformer_engine/pytorch/ops/basic/bias.py).
#include <cuda_bf16.h>
#include "launch.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace kb {

constexpr int LN_THREADS = 256;

__device__ __forceinline__ float ln_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float ln_block_sum(float v, float* red) {
  v = ln_warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < LN_THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) t = ln_warp_sum(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}

// one CTA per row (grid-stride); rows are re-read from L1/L2 in the second pass
__global__ void __launch_bounds__(LN_THREADS)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                     float* __restrict__ rstd, int rows, int H, float eps) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) s += __bfloat162float(xr[c]);
    const float mu = ln_block_sum(s, red) / H;
    float v = 0.f;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
      const float d = __bfloat162float(xr[c]) - mu;
      v += d * d;
    }
    const float r = rsqrtf(ln_block_sum(v, red) / H + eps);
    if (threadIdx.x == 0) {
      mean[row] = mu;
      rstd[row] = r;
    }
    __nv_bfloat16* yr = y + static_cast<size_t>(row) * H;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
      const float o = (__bfloat162float(xr[c]) - mu) * r * __bfloat162float(w[c]) + (b ? __bfloat162float(b[c]) : 0.f);
      yr[c] = __float2bfloat16(o);
    }
  }
}

// dx per row; per-CTA partial sums of dw and db into partial[grid][2][H]
__global__ void __launch_bounds__(LN_THREADS)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const float* __restrict__ mean, const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int H) {
  __shared__ float red[32];
  float* pw = partial + static_cast<size_t>(blockIdx.x) * 2 * H;
  float* pb = pw + H;
  for (int c = threadIdx.x; c < H; c += LN_THREADS) {
    pw[c] = 0.f;
    pb[c] = 0.f;
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t o = static_cast<size_t>(row) * H;
    const float mu = mean[row], r = rstd[row];
    float sg = 0.f, sgx = 0.f;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
      const float xh = (__bfloat162float(x[o + c]) - mu) * r;
      const float g = __bfloat162float(dy[o + c]) * __bfloat162float(w[c]);
      sg += g;
      sgx += g * xh;
    }
    const float mg = ln_block_sum(sg, red) / H;
    const float mgx = ln_block_sum(sgx, red) / H;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
      const float xh = (__bfloat162float(x[o + c]) - mu) * r;
      const float gy = __bfloat162float(dy[o + c]);
      const float g = gy * __bfloat162float(w[c]);
      dx[o + c] = __float2bfloat16((g - mg - xh * mgx) * r);
      pw[c] += gy * xh;      // each thread owns its columns of this CTA's partial rows
      pb[c] += gy;
    }
  }
}

__global__ void ln_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, float* __restrict__ db,
                                 int nparts, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float a = 0.f, b = 0.f;
  for (int p = 0; p < nparts; ++p) {
    a += partial[static_cast<size_t>(p) * 2 * H + c];
    b += partial[static_cast<size_t>(p) * 2 * H + H + c];
  }
  dw[c] = a;
  if (db) db[c] = b;
}

__global__ void bias_add_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long rows, int H) {
  const long total = rows * H;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16(__bfloat162float(x[i]) + __bfloat162float(b[i % H]));
}

// db[c] += sum over rows of dy[r][c]  (fp32 atomics; db zeroed or accumulated by the caller)
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ db, long rows, int H,
                              int rows_per_block) {
  const long r0 = static_cast<long>(blockIdx.y) * rows_per_block;
  const long r1 = min(rows, r0 + rows_per_block);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < H; c += gridDim.x * blockDim.x) {
    float s = 0.f;
    for (long r = r0; r < r1; ++r) s += __bfloat162float(dy[r * H + c]);
    atomicAdd(db + c, s);
  }
}

}  // namespace kb

using namespace kb;
#define LN_RET() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 2000 + (int)e_; } while (0)

extern "C" int kb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows,
                                int H, float eps, cudaStream_t st) {
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  KB_LAUNCH(layernorm_fwd_kernel, grid, LN_THREADS, 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                    (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, rows, H, eps);
  LN_RET();
}
extern "C" long kb_layernorm_bwd_scratch_elems(int rows, int H) {
  const int grid = rows < 148 * 2 ? rows : 148 * 2;
  return (long)grid * 2 * H;
}
extern "C" int kb_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* w,
                                void* dx, float* dw, float* db, float* scratch, int rows, int H, cudaStream_t st) {
  const int grid = rows < 148 * 2 ? rows : 148 * 2;
  KB_LAUNCH(layernorm_bwd_kernel, grid, LN_THREADS, 0, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean, rstd,
                                                    (const __nv_bfloat16*)w, (__nv_bfloat16*)dx, scratch, rows, H);
  KB_LAUNCH(ln_reduce_kernel, (H + 255) / 256, 256, 0, st, scratch, dw, db, grid, H);
  LN_RET();
}
extern "C" int kb_bias_add(const void* x, const void* b, void* y, long rows, int H, cudaStream_t st) {
  long blocks = (rows * H + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  KB_LAUNCH(bias_add_kernel, (int)blocks, 256, 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, rows, H);
  LN_RET();
}
extern "C" int kb_colsum_accumulate(const void* dy, float* db, long rows, int H, cudaStream_t st) {
  const int rpb = 256;
  dim3 grid((H + 255) / 256, (unsigned)((rows + rpb - 1) / rpb));
  KB_LAUNCH(colsum_kernel, grid, 256, 0, st, (const __nv_bfloat16*)dy, db, rows, H, rpb);
  LN_RET();
}
