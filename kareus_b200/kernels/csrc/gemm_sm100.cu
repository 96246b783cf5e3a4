// bf16 GEMM for sm_100a: C[M,N] (+)= A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer   (cp.async.bulk.tensor into a 4-stage, 128B-swizzled smem ring)
//   warp 1      MMA issuer     (tcgen05.mma 128xBNx16, one thread; TMEM allocation)
//   warps 2..5  epilogue       (tcgen05.ld of the accumulator, convert, store / accumulate)
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
// Both operands may be K-major (row = output index, K contiguous) or MN-major (row = K, output
// index contiguous), which covers fprop (x·Wᵀ), dgrad (dy·W) and wgrad (dyᵀ·x) without
// transposing anything in memory.  This is the role of the reference's cuBLASLt wrapper
// (3rdparty/TransformerEngine/transformer_engine/common/gemm/cublaslt_gemm.cu; layouts TN/NN/NT
// at kareus/transformer_engine/pytorch/ops/basic/basic_linear.py:572-582,848-859,899-909).
#include "sm100.cuh"
#include "launch.h"
#include "host_utils.h"
#include <stdlib.h>

namespace kb {

int gemm256_dispatch(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int lda, int b_mn, int ldb,
                     int ldc, int out_f32, int accumulate, int num_sms, int ks, int* status, cudaStream_t stream);

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGE_BYTES * GEMM_STAGES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 4 * 4096 + 1024;  // + epilogue staging + alignment slack
};

// Tile rasterisation: m-tiles are taken in groups of `group_m`; inside a group the m index runs
// fastest.  The 148 tiles in flight then cover a near-square patch of C whose A and B panels fit in
// L2 together, instead of streaming the whole of A once per wave.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = min(group_m, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Optional epilogue on the fp32 accumulator before it is stored: + bias[col] (bf16, per output
// feature) and then an activation (1: GELU, tanh approximation).  This is the fused forward of
// Linear + Bias (+ activation) of the reference's operator set
// (kareus/transformer_engine/pytorch/ops/basic/basic_linear_bias.py:34-315,
// ops/fused/forward_linear_bias_activation.py:37-213); Llama layers have no bias and pass null.
struct Epilogue {
  const __nv_bfloat16* bias;
  int act;
};
__device__ __forceinline__ void apply_epilogue(uint32_t (&v)[32], const Epilogue& ep, int col0, int N) {
  if (ep.bias == nullptr && ep.act == 0) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float x = __uint_as_float(v[j]);
    if (ep.bias != nullptr && col0 + j < N) x += __bfloat162float(ep.bias[col0 + j]);
    if (ep.act == 1) x = 0.5f * x * (1.f + tanhf(0.7978845608028654f * x * (1.f + 0.044715f * x * x)));
    v[j] = __float_as_uint(x);
  }
}

template <int BN, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 void* __restrict__ Cout, int M, int N, int K, int ldc, int group_m, int ks, int* status,
                 Epilogue ep) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::TILE_BYTES);
  uint64_t* empty = full + GEMM_STAGES;
  uint64_t* tfull = empty + GEMM_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int nk = (K + GEMM_BK - 1) / GEMM_BK;
  // split-K (accumulating outputs only): unit u = (tile u / ks, K part u % ks); every part adds its
  // partial sum to C with vector reductions, so parts of one tile may run on different SMs at once
  const int num_units = num_tiles * ks;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < GEMM_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        int tm, tn;
        tile_coords(u / ks, tiles_m, tiles_n, group_m, tm, tn);
        const int m0 = tm * GEMM_BM;
        const int n0 = tn * BN;
        const int kb0 = split_begin(nk, ks, u % ks), kb1 = split_begin(nk, ks, u % ks + 1);
        for (int kb_ = kb0; kb_ < kb1; ++kb_, ++it) {
          const int s = it % GEMM_STAGES;
          const uint32_t ph = (it / GEMM_STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          const int k0 = kb_ * GEMM_BK;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full[s], m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full[s], n0 + 64 * j, k0);
          }
        }
      }
      if (!ok) {
        // leave no copy in flight: tile loads land within microseconds, give them 200 us
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
    uint32_t it = 0;
    uint32_t tile_i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_i) {
      const uint32_t buf = tile_i & 1u;
      const uint32_t bph = (tile_i >> 1) & 1u;
      if (!mbar_wait(&tempty[buf], bph ^ 1u, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      const int kb0 = split_begin(nk, ks, u % ks), kb1 = split_begin(nk, ks, u % ks + 1);
      for (int kb_ = kb0; kb_ < kb1; ++kb_, ++it) {
        const int s = it % GEMM_STAGES;
        const uint32_t ph = (it / GEMM_STAGES) & 1u;
        if (!mbar_wait(&full[s], ph, abort_flag, status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc(a_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024)
                                     : make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_ss(d_tmem, ad, bd, idesc, (kb_ > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);                       // stage reusable once these MMAs retire
          if (kb_ == kb1 - 1) umma_commit(&tfull[buf]); // accumulator complete
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    uint32_t tile_i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_i) {
      const uint32_t buf = tile_i & 1u;
      const uint32_t bph = (tile_i >> 1) & 1u;
      int tm, tn;
      tile_coords(u / ks, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * GEMM_BM;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull[buf], bph, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
      if constexpr (!OUT_F32) {
        // bf16 output with 16-byte aligned rows: go through this warp's 4 KB of shared memory (32 rows
        // x 128 B, 16-byte units XOR-swizzled by row) so every store instruction writes four full
        // 128-byte row segments instead of 32 scattered 16-byte pieces
        if ((ldc & 7) == 0 && (N & 7) == 0) {
          uint8_t* stg = smem + S::TILE_BYTES + S::BAR_BYTES + q * 4096;
          __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(m0 + q * 32) * ldc;
#pragma unroll 1
          for (int cp = 0; cp < BN / 64; ++cp) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t v[32];
              tmem_ld_32x32(taddr + (cp * 2 + half) * 32, v);
              tmem_ld_wait();
              apply_epilogue(v, ep, n0 + cp * 64 + half * 32, N);
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
              if (m0 + q * 32 + r < M && col + 8 <= N)
                *reinterpret_cast<uint4*>(cbase + static_cast<size_t>(r) * ldc + col) = o;
            }
            __syncwarp();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[buf]);
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if constexpr (!ACCUM) apply_epilogue(v, ep, col, N);
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
                  float4 old = *p;
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- host side
template <int BN, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                       int num_sms, int ks, int* status, cudaStream_t stream, Epilogue ep) {
  CUtensorMap tmA, tmB;
  int rc;
  // K-major operand: dims (K, rows), box (64, tile rows).  MN-major: dims (rows, K), box (64, 64).
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, GEMM_BK, GEMM_BM);
  else       rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, 64, GEMM_BK);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, GEMM_BK, BN);
  else       rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, GEMM_BK);
  if (rc) return rc;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT_F32, ACCUM>;
  constexpr int smem = GemmSmem<BN>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    configured = true;
  }
  if (!ACCUM || ks < 1) ks = 1;
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN) * ks;
  int grid = tiles < num_sms ? tiles : num_sms;
  if (grid < 1) grid = 1;
  // m-tiles per group: keep the group's A panel near 40 MB so A and B panels share the 126 MB L2
  int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  long panel = (long)GEMM_BM * K * 2;
  int group_m = (int)((40L << 20) / (panel > 0 ? panel : 1));
  if (group_m < 4) group_m = 4;
  if (group_m > tiles_m) group_m = tiles_m;
  KB_LAUNCH(kern, grid, GEMM_THREADS, smem, stream, tmA, tmB, C, M, N, K, ldc, group_m, ks, status, ep);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

template <int BN, bool A_MN, bool B_MN>
static int dispatch_out(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                        int out_f32, int accumulate, int num_sms, int ks, int* status, cudaStream_t stream,
                        Epilogue ep) {
  if (out_f32 && accumulate)
    return launch_gemm<BN, A_MN, B_MN, true, true>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, ks, status, stream, ep);
  if (out_f32)
    return launch_gemm<BN, A_MN, B_MN, true, false>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, 1, status, stream, ep);
  if (accumulate) return ST_BAD_ARG;
  return launch_gemm<BN, A_MN, B_MN, false, false>(A, B, C, M, N, K, lda, ldb, ldc, num_sms, 1, status, stream, ep);
}

// ----------------------------------------------------------------------------- split-K choice
// Modelled time of an accumulating GEMM in units of one 64-deep K step of a 128x256 tile (~0.4 us):
// `waves` rounds of one unit each; a unit costs its K steps plus a fixed part (pipeline fill, epilogue,
// and with ks > 1 the reductions that every part sends to C).  Constants fitted to a sweep over the
// weight-gradient shapes of a 3B Llama layer at tensor-parallel sizes 1, 2 and 8 on a B200:
//   step   1.0 (128x256), 0.6 (128x128), 1.85 (256x256: twice the FLOPs, a little less L2 traffic per
//          FLOP)
//   fixed  14 + 2 ks (128-row tiles), 26 + 3 ks (256x256)
static inline double model_time(long tiles, int ks, int nk, int grid, double step, double fixed0, double fixed_ks) {
  const long units = tiles * ks;
  const long waves = (units + grid - 1) / grid;
  return waves * (static_cast<double>((nk + ks - 1) / ks) * step + fixed0 + fixed_ks * ks);
}

struct SplitChoice {
  int ks;
  double time;
};
static SplitChoice choose_split(long tiles, int nk, int grid, double step, double fixed0, double fixed_ks) {
  static const bool allow = [] { const char* e = getenv("KB_GEMM_SPLITK"); return !(e && e[0] == '0'); }();
  SplitChoice best{1, model_time(tiles, 1, nk, grid, step, fixed0, fixed_ks)};
  if (!allow) return best;
  for (int ks = 2; ks <= 8; ++ks) {
    if (nk / ks < 8) break;
    const double t = model_time(tiles, ks, nk, grid, step, fixed0, fixed_ks);
    if (t < best.time * 0.97) best = SplitChoice{ks, t};       // a split must pay for its extra traffic
  }
  return best;
}

// Accumulating output (weight gradients: few tiles, long K): tile and K split by modelled time.
struct AccumPlan {
  bool tile256;
  int ks;
};
static int g_force_tile = 0, g_force_ks = 0;   // measurement override, see kb_gemm_accum_force
static AccumPlan plan_accumulate(int M, int N, int K, int num_sms, bool fits256) {
  const int nk = (K + GEMM_BK - 1) / GEMM_BK;
  if (g_force_ks > 0) {
    const int ks = g_force_ks <= nk ? g_force_ks : nk;
    return AccumPlan{g_force_tile == 256 && fits256, ks};
  }
  const bool narrow = (N <= 128) || (N % 256 != 0 && N % 256 <= 128);
  const int bn = narrow ? 128 : 256;
  const long tiles128 = (long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + bn - 1) / bn);
  const SplitChoice c128 = choose_split(tiles128, nk, num_sms, narrow ? 0.6 : 1.0, 14.0, 2.0);
  if (fits256) {
    const long tiles256 = (long)((M + 255) / 256) * ((N + 255) / 256);
    const SplitChoice c256 = choose_split(tiles256, nk, num_sms, 1.85, 26.0, 3.0);
    if (c256.time < c128.time) return AccumPlan{true, c256.ks};
  }
  return AccumPlan{false, c128.ks};
}

}  // namespace kb

// Tile (128 or 256 rows) and K split that kb_gemm_bf16 uses for an accumulating fp32 output of this shape.
extern "C" void kb_gemm_accum_plan(int M, int N, int K, int num_sms, int* tile_rows, int* ks) {
  const bool fits256 = M >= 512 && N >= 512 && K >= 2048 && (N % 256 == 0 || N >= 4096);
  const kb::AccumPlan pl = kb::plan_accumulate(M, N, K, num_sms, fits256);
  *tile_rows = pl.tile256 ? 256 : 128;
  *ks = pl.ks;
}

// Measurement aid: force the tile (128 / 256) and K split of accumulating GEMMs; ks = 0 returns to the model.
extern "C" void kb_gemm_accum_force(int tile_rows, int ks) {
  kb::g_force_tile = tile_rows;
  kb::g_force_ks = ks;
}

// C[M,N] (+)= op(A) * op(B)^T.
//   a_mn = 0: A is [M, K] row-major (lda = row stride in elements); a_mn = 1: A is stored [K, M].
//   b_mn = 0: B is [N, K] row-major;                                b_mn = 1: B is stored [K, N].
//   out_f32: C is fp32 (else bf16); accumulate: C += (fp32 only).  num_sms limits the grid.
// Strides must be multiples of 8 elements and base pointers 16-byte aligned (TMA rules).
// kb_gemm_bias_act_bf16 adds the epilogue: bias (bf16 [N], may be null) and act (0 none, 1 GELU); it is not
// available together with accumulate.
extern "C" int kb_gemm_bias_act_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int lda,
                                     int b_mn, int ldb, int ldc, int out_f32, int accumulate, int num_sms,
                                     const void* bias, int act, int* status, cudaStream_t stream) {
  using namespace kb;
  if (M <= 0 || N <= 0 || K <= 0) return ST_BAD_ARG;
  if ((bias != nullptr || act != 0) && accumulate) return ST_BAD_ARG;
  if (act < 0 || act > 1) return ST_BAD_ARG;
  const Epilogue ep{reinterpret_cast<const __nv_bfloat16*>(bias), act};
  const bool plain = bias == nullptr && act == 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return ST_BAD_ARG;
  if (num_sms <= 0) num_sms = device_sm_count();
  int ks = 1;
  {
    // large problems with a long K loop: 256x256 tile per SM (a third less L2 traffic per FLOP; its
    // epilogue is not overlapped, which only pays off when the main loop is long), see gemm256_sm100.cu
    static const bool allow256 = [] { const char* e = getenv("KB_GEMM256"); return !(e && e[0] == '0'); }();
    const long tiles256 = (long)((M + 255) / 256) * ((N + 255) / 256);
    const bool fits256 = plain && allow256 && M >= 512 && N >= 512 && K >= 2048 && (N % 256 == 0 || N >= 4096);
    if (fits256 && !(out_f32 && accumulate) && tiles256 >= num_sms)
      return gemm256_dispatch(A, B, C, M, N, K, a_mn, lda, b_mn, ldb, ldc, out_f32, accumulate, num_sms, 1, status,
                              stream);
    if (out_f32 && accumulate) {
      const AccumPlan pl = plan_accumulate(M, N, K, num_sms, fits256);
      ks = pl.ks;
      if (pl.tile256)
        return gemm256_dispatch(A, B, C, M, N, K, a_mn, lda, b_mn, ldb, ldc, out_f32, accumulate, num_sms, pl.ks,
                                status, stream);
    }
  }
  // narrow outputs waste less of the last wave with the 128-wide tile
  const bool narrow = (N <= 128) || (N % 256 != 0 && N % 256 <= 128);
#define KB_GO(BN_)                                                                                         \
  do {                                                                                                     \
    if (!a_mn && !b_mn) return dispatch_out<BN_, false, false>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, accumulate, num_sms, ks, status, stream, ep); \
    if (!a_mn && b_mn) return dispatch_out<BN_, false, true>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, accumulate, num_sms, ks, status, stream, ep);   \
    if (a_mn && !b_mn) return dispatch_out<BN_, true, false>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, accumulate, num_sms, ks, status, stream, ep);   \
    return dispatch_out<BN_, true, true>(A, B, C, M, N, K, lda, ldb, ldc, out_f32, accumulate, num_sms, ks, status, stream, ep);                       \
  } while (0)
  if (narrow) KB_GO(128);
  KB_GO(256);
#undef KB_GO
}

extern "C" int kb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int lda,
                            int b_mn, int ldb, int ldc, int out_f32, int accumulate, int num_sms, int* status,
                            cudaStream_t stream) {
  return kb_gemm_bias_act_bf16(A, B, C, M, N, K, a_mn, lda, b_mn, ldb, ldc, out_f32, accumulate, num_sms, nullptr, 0,
                               status, stream);
}
