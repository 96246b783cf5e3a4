// bf16 GEMM with a 256x256 tile per SM (two 128x256 tcgen05 accumulators that share every B tile).
//
// Why: with a 128x256 tile each 64-deep K step pulls 48 KB from L2 for 512 tensor-core clocks; the
// profiler shows the tensor pipe ~73 % busy with L2 → shared-memory traffic as the limiter.  A
// 256x256 tile pulls 64 KB per 1024 clocks, a third less traffic per FLOP.  The two accumulators
// fill all 512 TMEM columns, so the epilogue of a tile is not overlapped with the next tile's main
// loop; with K >= 1024 that costs a few percent and the traffic saving wins.  Used for large
// problems (kb_gemm_bf16 picks it); same operand layouts as gemm_sm100.cu.
#include "sm100.cuh"
#include "launch.h"
#include "host_utils.h"

namespace kb {

constexpr int G2_BM = 256;
constexpr int G2_BN = 256;
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 3;
constexpr int G2_EPI_WARPS = 8;                 // 4 TMEM lane quarters x the 2 accumulators
constexpr int G2_THREADS = (2 + G2_EPI_WARPS) * 32;
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;   // 32 KB
constexpr int G2_B_BYTES = G2_BN * G2_BK * 2;   // 32 KB
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_TILE_BYTES = G2_STAGE_BYTES * G2_STAGES;
constexpr int G2_SMEM = G2_TILE_BYTES + 256 + G2_EPI_WARPS * 4096 + 1024;   // + per-warp epilogue staging

__device__ __forceinline__ void g2_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = min(group_m, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(G2_THREADS, 1)
gemm256_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    void* __restrict__ Cout, int M, int N, int K, int ldc, int group_m, int ks, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + G2_TILE_BYTES);
  uint64_t* empty = full + G2_STAGES;
  uint64_t* tfull = empty + G2_STAGES;
  uint64_t* tempty = tfull + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + G2_BM - 1) / G2_BM;
  const int tiles_n = (N + G2_BN - 1) / G2_BN;
  const int num_tiles = tiles_m * tiles_n;
  const int nk = (K + G2_BK - 1) / G2_BK;
  const int num_units = num_tiles * ks;   // split-K over accumulating outputs, as in gemm_sm100.cu

  if (threadIdx.x == 0) {
    for (int i = 0; i < G2_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, G2_EPI_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        int tm, tn;
        g2_tile_coords(u / ks, tiles_m, tiles_n, group_m, tm, tn);
        const int m0 = tm * G2_BM, n0 = tn * G2_BN;
        const int kb0 = split_begin(nk, ks, u % ks), kb1 = split_begin(nk, ks, u % ks + 1);
        for (int kb_ = kb0; kb_ < kb1; ++kb_, ++it) {
          const int s = it % G2_STAGES;
          const uint32_t ph = (it / G2_STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * G2_STAGE_BYTES;
          uint8_t* b_dst = a_dst + G2_A_BYTES;
          mbar_expect_tx(&full[s], G2_STAGE_BYTES);
          const int k0 = kb_ * G2_BK;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full[s], k0, m0);                         // [256 rows][64 k]
          } else {
#pragma unroll
            for (int j = 0; j < G2_BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full[s], m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < G2_BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full[s], n0 + 64 * j, k0);
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_bf16(128, G2_BN, A_MN, B_MN);
    uint32_t it = 0, tile_i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_i) {
      if (!mbar_wait(tempty, (tile_i & 1u) ^ 1u, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const int kb0 = split_begin(nk, ks, u % ks), kb1 = split_begin(nk, ks, u % ks + 1);
      for (int kb_ = kb0; kb_ < kb1; ++kb_, ++it) {
        const int s = it % G2_STAGES;
        const uint32_t ph = (it / G2_STAGES) & 1u;
        if (!mbar_wait(&full[s], ph, abort_flag, status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * G2_STAGE_BYTES);
          const uint32_t b_addr = a_addr + G2_A_BYTES;
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc(b_addr + k * 32, 16, 1024);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // rows h*128 .. h*128+127 of the A tile: K-major → 128 rows x 128 B further on;
              // MN-major → two 64-wide chunks (2 x 8 KB) further on
              const uint64_t ad = A_MN ? make_smem_desc(a_addr + h * 16384 + k * 2048, 8192, 1024)
                                       : make_smem_desc(a_addr + h * 16384 + k * 32, 16, 1024);
              umma_ss(tmem_base + h * G2_BN, ad, bd, idesc, (kb_ > kb0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(&empty[s]);
          if (kb_ == kb1 - 1) umma_commit(tfull);
        }
        __syncwarp();
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tile_i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_i) {
      int tm, tn;
      g2_tile_coords(u / ks, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * G2_BM, n0 = tn * G2_BN;
      if (!mbar_wait(tfull, tile_i & 1u, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // warps 2..5 read the accumulator of rows 0..127, warps 6..9 that of rows 128..255: two warps per
      // scheduler, so one warp's TMEM loads and conversions hide behind the other's stores
      {
        const int h = (warp - 2) >> 2;
        const int row = m0 + h * 128 + q * 32 + lane;
        const uint32_t taddr = tmem_base + h * G2_BN + (static_cast<uint32_t>(q * 32) << 16);
        bool stored = false;
        if constexpr (!OUT_F32) {
          // bf16 rows go through 4 KB of shared memory per warp so that stores are full 128-byte row
          // segments (see gemm_sm100.cu)
          if ((ldc & 7) == 0 && (N & 7) == 0) {
            uint8_t* stg = smem + G2_TILE_BYTES + 256 + (warp - 2) * 4096;
            __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(m0 + h * 128 + q * 32) * ldc;
#pragma unroll 1
            for (int cp = 0; cp < G2_BN / 64; ++cp) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + (cp * 2 + half) * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                  o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                  o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                  o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                  const int unit = half * 4 + j;
                  *reinterpret_cast<uint4*>(stg + lane * 128 + ((unit ^ (lane & 7)) << 4)) = o;
                }
              }
              __syncwarp();
              const int u = lane & 7;
              const int col = n0 + cp * 64 + u * 8;
#pragma unroll
              for (int it4 = 0; it4 < 8; ++it4) {
                const int r = it4 * 4 + (lane >> 3);
                const uint4 o = *reinterpret_cast<const uint4*>(stg + r * 128 + ((u ^ (r & 7)) << 4));
                if (m0 + h * 128 + q * 32 + r < M && col + 8 <= N)
                  *reinterpret_cast<uint4*>(cbase + static_cast<size_t>(r) * ldc + col) = o;
              }
              __syncwarp();
            }
            stored = true;
          }
        }
#pragma unroll 1
        for (int c = 0; c < (stored ? 0 : G2_BN / 32); ++c) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (row < M && col < N) {
            if constexpr (OUT_F32) {
              float* crow = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * ldc + col;
              if (col + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float4 o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                         __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                  float4* p = reinterpret_cast<float4*>(crow) + j;
                  if constexpr (ACCUM) {
                    if (ks > 1) { red_add_f32x4(p, o); continue; }
                    const float4 old = *p;
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                  }
                  *p = o;
                }
              } else {
                for (int j = 0; j < 32 && col + j < N; ++j) {
                  float o = __uint_as_float(v[j]);
                  if constexpr (ACCUM) {
                    if (ks > 1) { atomicAdd(crow + j, o); continue; }
                    o += crow[j];
                  }
                  crow[j] = o;
                }
              }
            } else {
              __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col;
              if (col + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                  o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                  o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                  o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                  reinterpret_cast<uint4*>(crow)[j] = o;
                }
              } else {
                for (int j = 0; j < 32 && col + j < N; ++j) crow[j] = __float2bfloat16(__uint_as_float(v[j]));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
static int launch256(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int num_sms,
                     int ks, int* status, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, G2_BK, G2_BM);
  else       rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, 64, G2_BK);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, G2_BK, G2_BN);
  else       rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, G2_BK);
  if (rc) return rc;
  auto kern = gemm256_bf16_kernel<A_MN, B_MN, OUT_F32, ACCUM>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM);
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    configured = true;
  }
  const int tiles_m = (M + G2_BM - 1) / G2_BM;
  if (!ACCUM || ks < 1) ks = 1;
  const int tiles = tiles_m * ((N + G2_BN - 1) / G2_BN) * ks;
  int grid = tiles < num_sms ? tiles : num_sms;
  long panel = (long)G2_BM * K * 2;
  int group_m = (int)((40L << 20) / (panel > 0 ? panel : 1));
  if (group_m < 2) group_m = 2;
  if (group_m > tiles_m) group_m = tiles_m;
  KB_LAUNCH(kern, grid, G2_THREADS, G2_SMEM, stream, tmA, tmB, C, M, N, K, ldc, group_m, ks, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

int gemm256_dispatch(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int lda, int b_mn, int ldb,
                     int ldc, int out_f32, int accumulate, int num_sms, int ks, int* status, cudaStream_t stream) {
#define G2_GO(AM, BM_)                                                                                          \
  do {                                                                                                          \
    if (out_f32 && accumulate) return launch256<AM, BM_, true, true>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, ks, status, stream);  \
    if (out_f32) return launch256<AM, BM_, true, false>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, ks, status, stream);               \
    return launch256<AM, BM_, false, false>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, ks, status, stream);                           \
  } while (0)
  if (!a_mn && !b_mn) G2_GO(false, false);
  if (!a_mn && b_mn) G2_GO(false, true);
  if (a_mn && !b_mn) G2_GO(true, false);
  G2_GO(true, true);
#undef G2_GO
}

}  // namespace kb
