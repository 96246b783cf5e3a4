// Memory-bound kernels of the Llama block and the optimizer, written for HBM3e: 16-byte vector
// accesses, one pass over the data, fp32 math in registers.
//   rmsnorm fwd/bwd      (reference path: TransformerEngine rmsnorm_fwd/bwd kernels)
//   rope (q and k in one launch, in place, strided views)  (reference: Apex fused RoPE)
//   swiglu fwd/bwd, dropout-add fwd/bwd, add (reference: torch.compile/Triton fused ops)
//   embedding gather / scatter-add, vocab-parallel cross entropy (reference: TE Triton CE)
//   fused AdamW over flat buffers, sum of squares (reference: TE/Apex multi_tensor kernels)
#include <cuda_bf16.h>
#include "launch.h"
#include "host_utils.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace kb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}
// One barrier per call: `red` holds two sets of 32 partial sums and consecutive calls alternate `parity`,
// so the next call's writes cannot overtake this call's reads (a thread reaches call n+2 only after the
// barrier of call n+1, which every thread passes after it has read the sums of call n).
template <int THREADS>
__device__ __forceinline__ float block_sum_alt(float v, float* red, int parity) {
  v = warp_sum(v);
  float* r = red + parity * 32;
  if ((threadIdx.x & 31) == 0) r[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += r[i];
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) t = warp_max(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}

struct bf8 { uint4 u; };
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ----------------------------------------------------------------------------- RMSNorm
// One CTA per row; H multiple of 8; each thread keeps up to VPT vectors of the row in registers.
constexpr int NORM_MAX_H = 256 * 4 * 8;   // widest row the register-resident kernels take (8192)

// THREADS x VPT vectors of 8 elements are kept in registers; the launcher picks the smallest variant that
// covers the row, so that narrow rows (3072: 384 threads x 1 vector) neither idle half of a 256-thread
// block nor carry register arrays sized for 8192-wide rows (which capped occupancy at 25 %).
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H, float eps) {
  constexpr int NORM_THREADS = THREADS;
  constexpr int NORM_VPT = VPT;
  __shared__ float red[64];
  const int nvec = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  // the next row's vectors are requested before this row's reduction, so a CTA always has a row in flight
  uint4 nx[NORM_VPT];
  if (blockIdx.x < rows) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(blockIdx.x) * H);
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) nx[i] = xr[v];
    }
  }
  int parity = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    uint4 xv[NORM_VPT];
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) xv[i] = nx[i];
    const int nrow = row + gridDim.x;
    if (nrow < rows) {
      const uint4* xn = reinterpret_cast<const uint4*>(x + static_cast<size_t>(nrow) * H);
#pragma unroll
      for (int i = 0; i < NORM_VPT; ++i) {
        const int v = threadIdx.x + i * NORM_THREADS;
        if (v < nvec) nx[i] = xn[v];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float f[8];
        unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
    }
    for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    const float tot = block_sum_alt<NORM_THREADS>(ss, red, parity);
    const float r = rsqrtf(tot / static_cast<float>(H) + eps);
    if (threadIdx.x == 0) rstd[row] = r;
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H);
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float f[8], g[8];
        unpack8(xv[i], f);
        unpack8(wr[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
        yr[v] = pack8(f);
      }
    }
    for (int v = threadIdx.x + NORM_VPT * NORM_THREADS; v < nvec; v += NORM_THREADS) {
      float f[8], g[8];
      unpack8(xr[v], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
      yr[v] = pack8(f);
    }
  }
}

// Narrow rows (per-head q/k norm, H <= 256): one warp per row.
__global__ void rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H,
                                        float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    float ss = 0.f;
    for (int c = lane; c < H; c += 32) {
      float v = __bfloat162float(xr[c]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / static_cast<float>(H) + eps);
    if (lane == 0) rstd[row] = r;
    for (int c = lane; c < H; c += 32)
      y[static_cast<size_t>(row) * H + c] = __float2bfloat16(__bfloat162float(xr[c]) * r * __bfloat162float(w[c]));
  }
}

// Backward: dx per row; dw partial sums per CTA into `partial[gridDim.x][H]` (scratch), reduced by
// rmsnorm_dw_reduce_kernel.  The grid is persistent (a few CTAs per SM) so `partial` stays small.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int H) {
  constexpr int NORM_THREADS = THREADS;
  constexpr int NORM_VPT = VPT;
  __shared__ float red[64];
  const int nvec = H >> 3;
  float dwacc[NORM_VPT][8];
#pragma unroll
  for (int i = 0; i < NORM_VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  // the next row's x and dy are requested before this row's reduction (see rmsnorm_fwd_kernel)
  uint4 nxx[NORM_VPT], nxg[NORM_VPT];
  float nr = 0.f;
  if (blockIdx.x < rows) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(blockIdx.x) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(blockIdx.x) * H);
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        nxx[i] = xr[v];
        nxg[i] = gr[v];
      }
    }
    nr = rstd[blockIdx.x];
  }
  int parity = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const float r = nr;
    float xh[NORM_VPT][8], g[NORM_VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(nxx[i], xf);
        unpack8(nxg[i], gf);
        unpack8(wr[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xf[j] * r;
          dwacc[i][j] += gf[j] * xh[i][j];
          g[i][j] = gf[j] * wf[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    const int nrow = row + gridDim.x;
    if (nrow < rows) {
      const uint4* xn = reinterpret_cast<const uint4*>(x + static_cast<size_t>(nrow) * H);
      const uint4* gn = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(nrow) * H);
#pragma unroll
      for (int i = 0; i < NORM_VPT; ++i) {
        const int v = threadIdx.x + i * NORM_THREADS;
        if (v < nvec) {
          nxx[i] = xn[v];
          nxg[i] = gn[v];
        }
      }
      nr = rstd[nrow];
    }
    const float c = block_sum_alt<NORM_THREADS>(dot, red, parity) / static_cast<float>(H);
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
#pragma unroll
    for (int i = 0; i < NORM_VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - xh[i][j] * c) * r;
        dr[v] = pack8(o);
      }
    }
  }
  float* prow = partial + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
  for (int i = 0; i < NORM_VPT; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) prow[v * 8 + j] = dwacc[i][j];
    }
  }
}

// `accumulate`: add the column sums to dw (the fp32 main gradient of the weight) instead of storing them.
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts,
                                         int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<size_t>(p) * H + c];
  dw[c] = accumulate ? dw[c] + s : s;
}

// General (slow) backward for narrow rows: one warp per row, dw via atomics.
__global__ void rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                        const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ w,
                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int rows, int H) {
  extern __shared__ float sdw[];
  for (int c = threadIdx.x; c < H; c += blockDim.x) sdw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const size_t o = static_cast<size_t>(row) * H;
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane; c < H; c += 32) {
      const float xh = __bfloat162float(x[o + c]) * r;
      const float g = __bfloat162float(dy[o + c]);
      atomicAdd(&sdw[c], g * xh);
      dot += g * __bfloat162float(w[c]) * xh;
    }
    dot = warp_sum(dot) / static_cast<float>(H);
    for (int c = lane; c < H; c += 32) {
      const float xh = __bfloat162float(x[o + c]) * r;
      const float g = __bfloat162float(dy[o + c]) * __bfloat162float(w[c]);
      dx[o + c] = __float2bfloat16((g - xh * dot) * r);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) atomicAdd(&dw[c], sdw[c]);
}

// ----------------------------------------------------------------------------- RoPE
// t is a strided view [s, b, g, rep, d]; one warp rotates one head vector (d = 128: 2 pairs/lane
// handled as one bf16x2 from each half).  cos/sin are [s, d/2] fp32 tables.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, long qs_s, long qs_b, long qs_g, long qs_r, int G, int R,
                            __nv_bfloat16* __restrict__ k, long ks_s, long ks_b, long ks_g, int KG,
                            const float* __restrict__ cosb, const float* __restrict__ sinb, int S, int B, int D,
                            float sign) {
  const int heads = G * R + KG;
  const long total = static_cast<long>(S) * B * heads;
  const int lane = threadIdx.x & 31;
  const int half = D >> 1;
  for (long wi = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wi < total;
       wi += (static_cast<long>(gridDim.x) * blockDim.x) >> 5) {
    const int h = static_cast<int>(wi % heads);
    const long sb = wi / heads;
    const int b = static_cast<int>(sb % B);
    const int s = static_cast<int>(sb / B);
    __nv_bfloat16* p;
    if (h < G * R) p = q + s * qs_s + b * qs_b + (h / R) * qs_g + (h % R) * qs_r;
    else p = k + s * ks_s + b * ks_b + (h - G * R) * ks_g;
    const float* cr = cosb + static_cast<long>(s) * half;
    const float* sr = sinb + static_cast<long>(s) * half;
    for (int i = lane * 2; i < half; i += 64) {
      __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(p + i);
      __nv_bfloat162 c = *reinterpret_cast<__nv_bfloat162*>(p + half + i);
      const float2 af = __bfloat1622float2(a), cf = __bfloat1622float2(c);
      const float c0 = cr[i], c1 = cr[i + 1], s0 = sr[i] * sign, s1 = sr[i + 1] * sign;
      // out1 = t1*cos - t2*sin ; out2 = t2*cos + t1*sin
      *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(af.x * c0 - cf.x * s0, af.y * c1 - cf.y * s1);
      *reinterpret_cast<__nv_bfloat162*>(p + half + i) =
          __floats2bfloat162_rn(cf.x * c0 + af.x * s0, cf.y * c1 + af.y * s1);
    }
  }
}

// Vectorised variant for head dims that are multiples of 16 (all models here: 128).  One warp owns one
// token (s, b): D/16 lanes form a group that rotates one head vector, 16 bytes from each half per lane,
// and the groups of the warp walk the token's heads.  The lane's 8 cos and 8 sin values are loaded once
// per token and stay in registers for all heads, so table traffic is amortised over the heads and every
// global access is a 16-byte vector.
__global__ void __launch_bounds__(256)
rope_vec_kernel(__nv_bfloat16* __restrict__ q, long qs_s, long qs_b, long qs_g, long qs_r, int G, int R,
                __nv_bfloat16* __restrict__ k, long ks_s, long ks_b, long ks_g, int KG,
                const float* __restrict__ cosb, const float* __restrict__ sinb, int S, int B, int D, float sign) {
  const int lanes_per_head = D >> 4;                 // 8 for D = 128
  const int groups = 32 / lanes_per_head;
  const int lane = threadIdx.x & 31;
  const int grp = lane / lanes_per_head;
  const int l = lane - grp * lanes_per_head;
  const int half = D >> 1;
  const int qh = G * R, heads = qh + KG;
  const long tokens = static_cast<long>(S) * B;
  for (long tok = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; tok < tokens;
       tok += (static_cast<long>(gridDim.x) * blockDim.x) >> 5) {
    const int b = static_cast<int>(tok % B);
    const int s = static_cast<int>(tok / B);
    float c[8], sn[8];
    {
      const float4* cr = reinterpret_cast<const float4*>(cosb + static_cast<long>(s) * half + l * 8);
      const float4* sr = reinterpret_cast<const float4*>(sinb + static_cast<long>(s) * half + l * 8);
      const float4 c0 = cr[0], c1 = cr[1], s0 = sr[0], s1 = sr[1];
      c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
      sn[0] = s0.x * sign; sn[1] = s0.y * sign; sn[2] = s0.z * sign; sn[3] = s0.w * sign;
      sn[4] = s1.x * sign; sn[5] = s1.y * sign; sn[6] = s1.z * sign; sn[7] = s1.w * sign;
    }
    __nv_bfloat16* qrow = q + s * qs_s + b * qs_b;
    __nv_bfloat16* krow = k + s * ks_s + b * ks_b;
#pragma unroll 2
    for (int h = grp; h < heads; h += groups) {
      __nv_bfloat16* p = h < qh ? qrow + (h / R) * qs_g + (h % R) * qs_r : krow + (h - qh) * ks_g;
      uint4* lo = reinterpret_cast<uint4*>(p + l * 8);
      uint4* hi = reinterpret_cast<uint4*>(p + half + l * 8);
      float a[8], d[8], o1[8], o2[8];
      unpack8(*lo, a);
      unpack8(*hi, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o1[i] = a[i] * c[i] - d[i] * sn[i];
        o2[i] = d[i] * c[i] + a[i] * sn[i];
      }
      *lo = pack8(o1);
      *hi = pack8(o2);
    }
  }
}

// ----------------------------------------------------------------------------- SwiGLU
// x [rows, 2F] = [gate | up]; y [rows, F]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows, int F) {
  const int fv = F >> 3;
  const long total = rows * fv;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / fv;
    const int c = static_cast<int>(i % fv);
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * 2 * F);
    float a[8], b[8];
    unpack8(xr[c], a);
    unpack8(xr[fv + c], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    reinterpret_cast<uint4*>(y + r * F)[c] = pack8(a);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                  __nv_bfloat16* __restrict__ dx, long rows, int F) {
  const int fv = F >> 3;
  const long total = rows * fv;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / fv;
    const int c = static_cast<int>(i % fv);
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * 2 * F);
    float a[8], b[8], g[8], da[8], db[8];
    unpack8(xr[c], a);
    unpack8(xr[fv + c], b);
    unpack8(reinterpret_cast<const uint4*>(dy + r * F)[c], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-a[j]));
      da[j] = g[j] * b[j] * s * (1.f + a[j] * (1.f - s));
      db[j] = g[j] * a[j] * s;
    }
    uint4* dr = reinterpret_cast<uint4*>(dx + r * 2 * F);
    dr[c] = pack8(da);
    dr[fv + c] = pack8(db);
  }
}

// ----------------------------------------------------------------------------- dropout-add / add
__device__ __forceinline__ uint32_t hash32(uint64_t idx, uint32_t seed) {
  // counter-based generator: two rounds of a 64-bit mix (splitmix64 finaliser)
  uint64_t z = idx + 0x9E3779B97F4A7C15ull * (static_cast<uint64_t>(seed) + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return static_cast<uint32_t>(z >> 32);
}
// y = residual + keep(x)/(1-p); one 8-vector per thread; the keep bit of element e is a pure
// function of (seed, e), so backward regenerates it.
__global__ void dropout_add_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                       __nv_bfloat16* __restrict__ y, long nvec, float p, uint32_t seed) {
  const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const uint32_t thr = static_cast<uint32_t>(p * 4294967296.0);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float a[8], r[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
    unpack8(reinterpret_cast<const uint4*>(res)[i], r);
    if (p > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = (hash32(static_cast<uint64_t>(i) * 8 + j, seed) >= thr) ? a[j] * scale : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += r[j];
    reinterpret_cast<uint4*>(y)[i] = pack8(a);
  }
}
__global__ void dropout_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, long nvec,
                                   float p, uint32_t seed) {
  const float scale = 1.f / (1.f - p);
  const uint32_t thr = static_cast<uint32_t>(p * 4294967296.0);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = (hash32(static_cast<uint64_t>(i) * 8 + j, seed) >= thr) ? a[j] * scale : 0.f;
    reinterpret_cast<uint4*>(dx)[i] = pack8(a);
  }
}
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, long nvec) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float x[8], z[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(b)[i], z);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += z[j];
    reinterpret_cast<uint4*>(y)[i] = pack8(x);
  }
}

// ----------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const long* __restrict__ tokens, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, long ntok, int H, long vocab_start, long vlocal) {
  const int hv = H >> 3;
  for (long t = blockIdx.x; t < ntok; t += gridDim.x) {
    const long id = tokens[t] - vocab_start;
    const bool inside = id >= 0 && id < vlocal;
    const uint4* src = reinterpret_cast<const uint4*>(w + (inside ? id : 0) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + t * H);
    for (int c = threadIdx.x; c < hv; c += blockDim.x) dst[c] = inside ? src[c] : make_uint4(0, 0, 0, 0);
  }
}
__global__ void embedding_bwd_kernel(const long* __restrict__ tokens, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ gw, long ntok, int H, long vocab_start, long vlocal) {
  for (long t = blockIdx.x; t < ntok; t += gridDim.x) {
    const long id = tokens[t] - vocab_start;
    if (id < 0 || id >= vlocal) continue;
    float* dst = gw + id * H;
    const __nv_bfloat16* src = dout + t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) atomicAdd(dst + c, __bfloat162float(src[c]));
  }
}

// ----------------------------------------------------------------------------- cross entropy
// Pass 1: per row (max, sum exp(x-max), target logit) over this rank's vocabulary shard.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long* __restrict__ targets, float* __restrict__ omax,
                float* __restrict__ osum, float* __restrict__ otgt, long rows, int V, long vocab_start) {
  __shared__ float red[32];
  const int vv = V >> 3;
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* lr = logits + row * V;
    const uint4* l4 = reinterpret_cast<const uint4*>(lr);
    float m = -INFINITY, s = 0.f;
    for (int c = threadIdx.x; c < vv; c += CE_THREADS) {
      float f[8];
      unpack8(l4[c], f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int c = (vv << 3) + threadIdx.x; c < V; c += CE_THREADS) {
      const float f = __bfloat162float(lr[c]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
    }
    const float gm = block_max<CE_THREADS>(m, red);
    const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum<CE_THREADS>(contrib, red);
    if (threadIdx.x == 0) {
      omax[row] = gm;
      osum[row] = gs;
      const long t = targets[row] - vocab_start;
      otgt[row] = (t >= 0 && t < V) ? __bfloat162float(lr[t]) : 0.f;
    }
  }
}
// Pass 2: logits := (softmax - onehot) * scale[row]  (in place)
__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ targets, const float* __restrict__ gmax,
               const float* __restrict__ gsum, const float* __restrict__ scale, long rows, int V, long vocab_start) {
  const int vv = V >> 3;
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* lr = logits + row * V;
    uint4* l4 = reinterpret_cast<uint4*>(lr);
    const float m = gmax[row], inv = 1.f / gsum[row], sc = scale[row];
    const long t = targets[row] - vocab_start;
    for (int c = threadIdx.x; c < vv; c += CE_THREADS) {
      float f[8];
      unpack8(l4[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - m) * inv;
        if (static_cast<long>(c) * 8 + j == t) p -= 1.f;
        f[j] = p * sc;
      }
      l4[c] = pack8(f);
    }
    for (int c = (vv << 3) + threadIdx.x; c < V; c += CE_THREADS) {
      float p = __expf(__bfloat162float(lr[c]) - m) * inv;
      if (c == t) p -= 1.f;
      lr[c] = __float2bfloat16(p * sc);
    }
  }
}

// ----------------------------------------------------------------------------- optimizer
// AdamW over flat buffers: fp32 master/m/v, fp32 grad, bf16 parameter written back.
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, float* __restrict__ master, long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, const float* __restrict__ grad_scale_ptr,
                             float grad_scale) {
  const float gs = grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale;
  const long n4 = n >> 2;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 ww = reinterpret_cast<float4*>(master)[i];
    float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x; float* wa = &ww.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = ga[j] * gs;
      ma[j] = b1 * ma[j] + (1.f - b1) * gr;
      va[j] = b2 * va[j] + (1.f - b2) * gr * gr;
      const float den = sqrtf(va[j] / bc2) + eps;
      wa[j] = wa[j] * (1.f - lr * wd) - lr * (ma[j] / bc1) / den;
    }
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    reinterpret_cast<float4*>(master)[i] = ww;
    if (p) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(ww.x, ww.y);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(ww.z, ww.w);
      reinterpret_cast<uint2*>(p)[i] = o;
    }
  }
  // tail
  for (long i = (n4 << 2) + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gr = g[i] * gs;
    const float mi = b1 * m[i] + (1.f - b1) * gr;
    const float vi = b2 * v[i] + (1.f - b2) * gr * gr;
    const float wi = master[i] * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    m[i] = mi; v[i] = vi; master[i] = wi;
    if (p) p[i] = __float2bfloat16(wi);
  }
}

// out[0] += sum(x^2)  (fp32 input); out must be zeroed by the caller.
__global__ void sumsq_f32_kernel(const float* __restrict__ x, long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const long n4 = n >> 2;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 t = reinterpret_cast<const float4*>(x)[i];
    s += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  for (long i = (n4 << 2) + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    s += x[i] * x[i];
  const float tot = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, tot);
}
__global__ void sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ x, long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float t = __bfloat162float(x[i]);
    s += t * t;
  }
  const float tot = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, tot);
}

// Variant of the RMSNorm kernels for a row of H elements: threads per CTA and vectors per thread.
struct NormVariant { int id, threads, vpt; };
static inline NormVariant norm_variant(int H) {
  const int nvec = H >> 3;
  if (nvec <= 128) return {0, 128, 1};
  if (nvec <= 256) return {1, 256, 1};
  if (nvec <= 384) return {2, 384, 1};
  if (nvec <= 512) return {3, 256, 2};
  return {4, 256, 4};
}
#define KB_NORM_DISPATCH(variant, CALL)           \
  switch ((variant).id) {                         \
    case 0: { CALL(128, 1); break; }              \
    case 1: { CALL(256, 1); break; }              \
    case 2: { CALL(384, 1); break; }              \
    case 3: { CALL(256, 2); break; }              \
    default: { CALL(256, 4); break; }             \
  }

// CTAs of `kern` that an SM holds at once (registers and threads), asked from the runtime.
template <typename Kern>
static int resident_ctas(Kern kern, int threads) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, 0) != cudaSuccess || n < 1) n = 1;
  return n;
}
// Persistent grid of the RMSNorm backward for rows of H elements (also the number of partial dw rows).
static int norm_bwd_ctas(int H) {
  static int cached[5] = {0, 0, 0, 0, 0};
  const NormVariant nv = norm_variant(H);
  if (cached[nv.id] == 0) {
    int per_sm = 1;
#define KB_OCC(T_, V_) per_sm = resident_ctas(rmsnorm_bwd_kernel<T_, V_>, T_)
    KB_NORM_DISPATCH(nv, KB_OCC)
#undef KB_OCC
    cached[nv.id] = device_sm_count() * per_sm;
  }
  return cached[nv.id];
}
static int norm_fwd_ctas(int H) {
  static int cached[5] = {0, 0, 0, 0, 0};
  const NormVariant nv = norm_variant(H);
  if (cached[nv.id] == 0) {
    int per_sm = 1;
#define KB_OCC(T_, V_) per_sm = resident_ctas(rmsnorm_fwd_kernel<T_, V_>, T_)
    KB_NORM_DISPATCH(nv, KB_OCC)
#undef KB_OCC
    cached[nv.id] = device_sm_count() * per_sm;
  }
  return cached[nv.id];
}

static inline int grid_for(long work, int threads, int max_blocks) {
  long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

}  // namespace kb

using namespace kb;
#define KB_CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 2000 + (int)e_; } while (0)

extern "C" int kb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H, float eps,
                              cudaStream_t st) {
  if (H % 8 == 0 && H >= 512) {
    const NormVariant nv = norm_variant(H);
    const int grid = grid_for(rows, 1, norm_fwd_ctas(H));          // one resident wave: rows are dealt evenly
#define KB_FWD(T_, V_)                                                                                            \
    KB_LAUNCH((rmsnorm_fwd_kernel<T_, V_>), grid, T_, 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,      \
              (__nv_bfloat16*)y, rstd, rows, H, eps)
    KB_NORM_DISPATCH(nv, KB_FWD)
#undef KB_FWD
  } else {
    KB_LAUNCH(rmsnorm_fwd_warp_kernel, grid_for(rows, 8, 148 * 8), 256, 0, st, 
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, H, eps);
  }
  KB_CHECK_LAUNCH();
}

// Number of fp32 elements of scratch that kb_rmsnorm_bwd needs for a given H (0 for narrow rows).
extern "C" long kb_rmsnorm_bwd_scratch_elems(int rows, int H) {
  if (H % 8 == 0 && H >= 512 && H <= NORM_MAX_H) return (long)grid_for(rows, 1, norm_bwd_ctas(H)) * H;
  return 0;
}

// dx and the weight gradient of RMSNorm.  accumulate = 0: dw receives the gradient; 1: the gradient is
// added to dw (callers pass the weight's fp32 main gradient and save a separate add).
extern "C" int kb_rmsnorm_bwd_acc(const void* dy, const void* x, const float* rstd, const void* w, void* dx, float* dw,
                                  float* scratch, int rows, int H, int accumulate, cudaStream_t st) {
  if (H % 8 == 0 && H >= 512 && H <= NORM_MAX_H) {
    const NormVariant nv = norm_variant(H);
    const int grid = grid_for(rows, 1, norm_bwd_ctas(H));          // must match kb_rmsnorm_bwd_scratch_elems
    if (!scratch) return 7;
#define KB_BWD(T_, V_)                                                                                              \
    KB_LAUNCH((rmsnorm_bwd_kernel<T_, V_>), grid, T_, 0, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd, \
              (const __nv_bfloat16*)w, (__nv_bfloat16*)dx, scratch, rows, H)
    KB_NORM_DISPATCH(nv, KB_BWD)
#undef KB_BWD
    KB_LAUNCH(rmsnorm_dw_reduce_kernel, (H + 255) / 256, 256, 0, st, scratch, dw, grid, H, accumulate);
  } else {
    if (!accumulate) kb::memset_async(dw, 0, sizeof(float) * H, st);    // the kernel adds with atomics
    KB_LAUNCH(rmsnorm_bwd_warp_kernel, grid_for(rows, 8, 148 * 4), 256, sizeof(float) * H, st, 
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd, (const __nv_bfloat16*)w, (__nv_bfloat16*)dx, dw,
        rows, H);
  }
  KB_CHECK_LAUNCH();
}

extern "C" int kb_rmsnorm_bwd(const void* dy, const void* x, const float* rstd, const void* w, void* dx, float* dw,
                              float* scratch, int rows, int H, cudaStream_t st) {
  return kb_rmsnorm_bwd_acc(dy, x, rstd, w, dx, dw, scratch, rows, H, 0, st);
}

extern "C" int kb_rope(void* q, long qs_s, long qs_b, long qs_g, long qs_r, int G, int R, void* k, long ks_s,
                       long ks_b, long ks_g, int KG, const float* cosb, const float* sinb, int S, int B, int D,
                       int inverse, cudaStream_t st) {
  if (D % 4) return 7;
  {
    // 16-byte vectors need 16-byte aligned head rows: every stride a multiple of 8 elements
    const bool al = ((qs_s | qs_b | qs_g | qs_r | ks_s | ks_b | ks_g) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (k == nullptr || (reinterpret_cast<uintptr_t>(k) & 15) == 0);
    if (al && D % 16 == 0 && D >= 16 && D <= 512 && (32 % (D / 16)) == 0) {
      const long tokens = (long)S * B;
      KB_LAUNCH(rope_vec_kernel, grid_for(tokens * 32, 256, 148 * 8), 256, 0, st,
          (__nv_bfloat16*)q, qs_s, qs_b, qs_g, qs_r, G, R, (__nv_bfloat16*)k, ks_s, ks_b, ks_g, KG, cosb, sinb, S, B, D,
          inverse ? -1.f : 1.f);
      KB_CHECK_LAUNCH();
    }
  }
  const long warps = (long)S * B * (G * R + KG);
  KB_LAUNCH(rope_kernel, grid_for(warps * 32, 256, 148 * 16), 256, 0, st, 
      (__nv_bfloat16*)q, qs_s, qs_b, qs_g, qs_r, G, R, (__nv_bfloat16*)k, ks_s, ks_b, ks_g, KG, cosb, sinb, S, B, D,
      inverse ? -1.f : 1.f);
  KB_CHECK_LAUNCH();
}

extern "C" int kb_swiglu_fwd(const void* x, void* y, long rows, int F, cudaStream_t st) {
  if (F % 8) return 7;
  KB_LAUNCH(swiglu_fwd_kernel, grid_for(rows * (F / 8), 256, 148 * 16), 256, 0, st, (const __nv_bfloat16*)x,
                                                                              (__nv_bfloat16*)y, rows, F);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_swiglu_bwd(const void* dy, const void* x, void* dx, long rows, int F, cudaStream_t st) {
  if (F % 8) return 7;
  KB_LAUNCH(swiglu_bwd_kernel, grid_for(rows * (F / 8), 256, 148 * 16), 256, 0, st, 
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, rows, F);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_dropout_add_fwd(const void* x, const void* res, void* y, long n, float p, unsigned seed,
                                  cudaStream_t st) {
  if (n % 8) return 7;
  KB_LAUNCH(dropout_add_fwd_kernel, grid_for(n / 8, 256, 148 * 16), 256, 0, st, 
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (__nv_bfloat16*)y, n / 8, p, seed);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_dropout_bwd(const void* dy, void* dx, long n, float p, unsigned seed, cudaStream_t st) {
  if (n % 8) return 7;
  KB_LAUNCH(dropout_bwd_kernel, grid_for(n / 8, 256, 148 * 16), 256, 0, st, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx,
                                                                      n / 8, p, seed);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_add(const void* a, const void* b, void* y, long n, cudaStream_t st) {
  if (n % 8) return 7;
  KB_LAUNCH(add_kernel, grid_for(n / 8, 256, 148 * 16), 256, 0, st, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                              (__nv_bfloat16*)y, n / 8);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_embedding_fwd(const long* tokens, const void* w, void* out, long ntok, int H, long vocab_start,
                                long vlocal, cudaStream_t st) {
  if (H % 8) return 7;
  KB_LAUNCH(embedding_fwd_kernel, grid_for(ntok, 1, 148 * 16), 128, 0, st, tokens, (const __nv_bfloat16*)w,
                                                                     (__nv_bfloat16*)out, ntok, H, vocab_start, vlocal);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_embedding_bwd(const long* tokens, const void* dout, float* gw, long ntok, int H, long vocab_start,
                                long vlocal, cudaStream_t st) {
  KB_LAUNCH(embedding_bwd_kernel, grid_for(ntok, 1, 148 * 16), 256, 0, st, tokens, (const __nv_bfloat16*)dout, gw, ntok, H,
                                                                     vocab_start, vlocal);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_ce_stats(const void* logits, const long* targets, float* omax, float* osum, float* otgt, long rows,
                           int V, long vocab_start, cudaStream_t st) {
  KB_LAUNCH(ce_stats_kernel, grid_for(rows, 1, 148 * 4), CE_THREADS, 0, st, (const __nv_bfloat16*)logits, targets, omax, osum,
                                                                      otgt, rows, V, vocab_start);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_ce_grad(void* logits, const long* targets, const float* gmax, const float* gsum, const float* scale,
                          long rows, int V, long vocab_start, cudaStream_t st) {
  KB_LAUNCH(ce_grad_kernel, grid_for(rows, 1, 148 * 4), CE_THREADS, 0, st, (__nv_bfloat16*)logits, targets, gmax, gsum, scale,
                                                                     rows, V, vocab_start);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_adamw(void* p, const float* g, float* m, float* v, float* master, long n, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale_ptr,
                        float grad_scale, cudaStream_t st) {
  KB_LAUNCH(adamw_kernel, grid_for(n / 4 + 1, 256, 148 * 16), 256, 0, st, (__nv_bfloat16*)p, g, m, v, master, n, lr, b1, b2,
                                                                    eps, wd, bc1, bc2, grad_scale_ptr, grad_scale);
  KB_CHECK_LAUNCH();
}
extern "C" int kb_sumsq(const void* x, long n, int is_f32, float* out, cudaStream_t st) {
  if (is_f32) KB_LAUNCH(sumsq_f32_kernel, grid_for(n / 4 + 1, 256, 148 * 8), 256, 0, st, (const float*)x, n, out);
  else KB_LAUNCH(sumsq_bf16_kernel, grid_for(n, 256, 148 * 8), 256, 0, st, (const __nv_bfloat16*)x, n, out);
  KB_CHECK_LAUNCH();
}

// ----------------------------------------------------------------------------- allocation-free RMSNorm backward
// Declared in kareus_b200_noalloc.h.  Same kernels as kb_rmsnorm_bwd; the per-CTA partial sums of
// the weight gradient live in a fixed device array instead of caller-provided scratch.
namespace kb {
constexpr int NOALLOC_MAX_H = 8192;
constexpr int NOALLOC_MAX_CTAS = 148;
static __device__ __align__(256) float g_rmsnorm_bwd_partial[NOALLOC_MAX_CTAS * NOALLOC_MAX_H];
static float* g_rmsnorm_bwd_partial_addr[64] = {nullptr};
}  // namespace kb

extern "C" int kb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* rstd, const void* w, void* dx,
                                      float* dw, int rows, int H, cudaStream_t st) {
  if (rows <= 0 || H < 512 || H > NOALLOC_MAX_H || (H % 8) != 0) return 7;   // outside the supported range
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 7;
  if (g_rmsnorm_bwd_partial_addr[dev] == nullptr) {
    // once per device, with that device current: the symbol's name is only a host-side handle,
    // the kernel needs the device address behind it
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_rmsnorm_bwd_partial);
    if (e != cudaSuccess || ptr == nullptr) return 1000 + static_cast<int>(e);
    g_rmsnorm_bwd_partial_addr[dev] = ptr;
  }
  float* partial = g_rmsnorm_bwd_partial_addr[dev];
  const int grid = rows < NOALLOC_MAX_CTAS ? rows : NOALLOC_MAX_CTAS;
  KB_LAUNCH((rmsnorm_bwd_kernel<256, 4>), grid, 256, 0, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd,
                                                    (const __nv_bfloat16*)w, (__nv_bfloat16*)dx, partial, rows, H);
  KB_LAUNCH(rmsnorm_dw_reduce_kernel, (H + 255) / 256, 256, 0, st, partial, dw, grid, H, 0);
  KB_CHECK_LAUNCH();
}
