// Causal GQA flash-attention forward for sm_100a, head dim 128, bf16 in / bf16 out, fp32 softmax.
//
// One CTA owns a tile of 128 query rows of one (batch, head) and walks the visible key tiles:
//   warp 0      TMA producer: Q once, then K and V tiles into a 2-stage ring (128B swizzle)
//   warp 1      MMA issuer:   S = Q·Kᵀ (tcgen05, accumulator in TMEM, double buffered) and
//                             O += P·V (P from shared memory, V as an MN-major operand)
//   warps 2..17 softmax:      four threads per query row, 32 key columns each (warp = TMEM lane quarter
//                             x column chunk): S from TMEM once, kept in registers → scale, mask, row
//                             maximum exchanged among the four threads through spare TMEM columns and a
//                             128-thread named barrier → P (bf16) into swizzled shared memory, partial
//                             row sums per thread.  Sixteen warps, four per scheduler: with one thread
//                             per row and one warp per scheduler the exponentials set the pace.
// The S of tile j+1 is issued before the softmax of tile j finishes, so tensor cores and the
// exponent units overlap.  O stays in TMEM for the whole row tile; it is rescaled only when the
// running maximum moves by more than 2^8 ("lazy rescale"), which happens on the first tiles only.
//
// Chunked keys (context parallelism without a gathered copy): the logical key sequence may be cut
// into equal chunks that live in different buffers — each context-parallel rank's K/V shard inside
// its own heap, reached through its peer mapping.  The producer picks the tensor map and the row
// inside it from a small chunk table (`ChunkGeom`), everything else works on logical key positions,
// so one launch covers what a ring of per-chunk launches plus log-sum-exp merges would compute
// (3rdparty/TransformerEngine/.../context_parallel.py:94-162,676-712).  Query rows may likewise be
// two chunks with their own absolute positions (dual-chunk causal load balance).  Remote tiles are
// fetched with plain (non-multicast) TMA loads.
//
// Q, K and V are read through TMA from strided views of the packed QKV projection
// ([s, b, groups, (rep+2)·d]), so no transpose or copy precedes the kernel (the reference
// transposes sbhd→bshd and calls the FlashAttention-2 wheel:
// kareus/transformer_engine/pytorch/attention/dot_product_attention/backends.py:179-186,328-333).
#include "sm100.cuh"
#include "launch.h"
#include "host_utils.h"
#include <string.h>

namespace kb {

constexpr int FA_BM = 128;      // query rows per CTA
constexpr int FA_BN = 128;      // keys per tile
constexpr int FA_D = 128;       // head dim
constexpr int FA_SOFTMAX_WARPS = 16;
constexpr int FA_THREADS = (2 + FA_SOFTMAX_WARPS) * 32;
constexpr int FA_TILE_BYTES = FA_BN * FA_D * 2;   // 32 KB: two 64-wide swizzled chunks of 16 KB
constexpr int FA_CHUNK = 16384;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

}  // namespace kb
#include "attention_chunks.h"
namespace kb {

struct FwdParams {
  __nv_bfloat16* out;   // [sq, b, hq, d] contiguous
  float* lse;           // [b, hq, sq]
  int sq, skv, b, hq, rep;
  int q_offset;         // absolute position of query row 0 relative to key 0
  float scale_log2;     // softmax scale * log2(e)
  int causal;
  int* status;
  ChunkGeom geom;       // chunk tables (all zero: one K/V buffer, one query chunk at q_offset)
};

constexpr int FA_KSTAGES = 2;   // K tiles are released as soon as their S MMA retires
constexpr int FA_VSTAGES = 2;   // V tiles after their P·V MMA

struct FaSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + FA_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + FA_KSTAGES * FA_TILE_BYTES;
  static constexpr int P_OFF = V_OFF + FA_VSTAGES * FA_TILE_BYTES;
  static constexpr int BAR_OFF = P_OFF + 2 * FA_TILE_BYTES;   // P is double buffered
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ KvMaps kv,
                      const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FaSmem::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [FA_KSTAGES]
  uint64_t* k_empty = bars + 4;   // [FA_KSTAGES]
  uint64_t* v_full = bars + 7;    // [2]
  uint64_t* v_empty = bars + 9;   // [2]
  uint64_t* s_full = bars + 11;   // [2]
  uint64_t* s_empty = bars + 13;  // [2]
  uint64_t* p_full = bars + 15;   // [2]
  uint64_t* pv_done = bars + 17;  // [2]  P·V of the tile that used P buffer b has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // heavy (late) query tiles first
  const int n_qtiles = (p.sq + FA_BM - 1) / FA_BM;
  const int qt = n_qtiles - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int g = head / p.rep, r = head % p.rep;
  const int q0 = qt * FA_BM;
  // absolute position of local query row x of this tile is q_off + x
  const int q_off = p.geom.q_offset_of(q0, p.q_offset);
  // keys visible to this tile: [0, kv_end)
  int kv_end = p.skv;
  if (p.causal) {
    const int last_q = q_off + min(q0 + FA_BM, p.sq) - 1;
    kv_end = min(p.skv, last_q + 1);
  }
  const int n_kv = kv_end > 0 ? (kv_end + FA_BN - 1) / FA_BN : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < FA_KSTAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], FA_SOFTMAX_WARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_full[i], FA_SOFTMAX_WARPS);
      mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;         // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;   // 128 columns
  const uint32_t tmem_x = tmem_base + 384;   // 12 columns: row maxima (2 x 4) and row sums (4) of the column chunks

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && n_kv > 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&kv.k[0]);
      prefetch_tmap(&kv.v[0]);
      mbar_expect_tx(q_full, FA_TILE_BYTES);
      tma_load_5d(smem + FaSmem::Q_OFF, &tmQ, q_full, 0, r, g, batch, q0);
      tma_load_5d(smem + FaSmem::Q_OFF + FA_CHUNK, &tmQ, q_full, 64, r, g, batch, q0);
      bool okp = true;
      auto load_k = [&](int j) {
        const int s = j % FA_KSTAGES;
        const uint32_t ph = (j / FA_KSTAGES) & 1u;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { okp = false; return; }
        uint8_t* kd = smem + FaSmem::K_OFF + s * FA_TILE_BYTES;
        mbar_expect_tx(&k_full[s], FA_TILE_BYTES);
        int src, srow;
        p.geom.locate(j * FA_BN, src, srow);
        tma_load_4d(kd, &kv.k[src], &k_full[s], 0, g, batch, srow);
        tma_load_4d(kd + FA_CHUNK, &kv.k[src], &k_full[s], 64, g, batch, srow);
      };
      load_k(0);
      // K runs one tile ahead of V: K(j+1) is requested before V(j)
      for (int j = 0; j < n_kv && okp; ++j) {
        if (j + 1 < n_kv) load_k(j + 1);
        if (!okp) break;
        const int s = j % FA_VSTAGES;
        const uint32_t ph = (j / FA_VSTAGES) & 1u;
        if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        uint8_t* vd = smem + FaSmem::V_OFF + s * FA_TILE_BYTES;
        mbar_expect_tx(&v_full[s], FA_TILE_BYTES);
        int src, srow;
        p.geom.locate(j * FA_BN, src, srow);
        tma_load_4d(vd, &kv.v[src], &v_full[s], 0, g, batch, srow);
        tma_load_4d(vd + FA_CHUNK, &kv.v[src], &v_full[s], 64, g, batch, srow);
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, FA_BN, false, false);  // Q K-major, K K-major
    constexpr uint32_t idesc_o = make_idesc_bf16(FA_BM, FA_D, false, true);    // P K-major, V MN-major
    const uint32_t q_addr = smem_u32(smem + FaSmem::Q_OFF);
    const uint32_t p_addr = smem_u32(smem + FaSmem::P_OFF);
    bool ok = n_kv > 0;
    auto issue_s = [&](int j) {
      const int s = j & 1;
      const int ks = j % FA_KSTAGES;
      const uint32_t k_addr = smem_u32(smem + FaSmem::K_OFF + ks * FA_TILE_BYTES);
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          const uint32_t off = (k >> 2) * FA_CHUNK + (k & 3) * 32;
          umma_ss(tmem_s + s * FA_BN, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024),
                  idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(&s_full[s]);
      }
      __syncwarp();
    };
    if (ok) ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL);
    if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, ST_TIMEOUT_FULL);
    if (ok) {
      tc_fence_after();
      issue_s(0);
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      if (j + 1 < n_kv) {
        const int s1 = (j + 1) & 1;
        const uint32_t ph1 = ((j + 1) >> 1) & 1u;
        if (!mbar_wait(&k_full[(j + 1) % FA_KSTAGES], ((j + 1) / FA_KSTAGES) & 1u, abort_flag, p.status,
                       ST_TIMEOUT_FULL)) { ok = false; break; }
        if (!mbar_wait(&s_empty[s1], ph1 ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_s(j + 1);
      }
      if (!mbar_wait(&p_full[s], (j >> 1) & 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      if (!mbar_wait(&v_full[s], (j >> 1) & 1u, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(smem + FaSmem::V_OFF + s * FA_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          // A = P [128 rows][128 keys] K-major: two 64-key chunks; B = V [keys][d] MN-major
          const uint32_t a_off = (k >> 2) * FA_CHUNK + (k & 3) * 32;
          umma_ss(tmem_o, make_smem_desc(p_addr + s * FA_TILE_BYTES + a_off, 16, 1024),
                  make_smem_desc(v_addr + k * 2048, FA_CHUNK, 1024), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(&pv_done[s]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;
    const int c = (warp - 2) >> 2;                 // chunk of 32 key columns, and of 32 output columns
    const int row = quarter * 32 + lane;           // row inside the tile = TMEM lane
    const int qpos = q_off + q0 + row;             // absolute position of this query
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int group_bar = 1 + quarter;             // named barrier of the four warps that share these rows
    const uint32_t full = 0xffffffffu;
    float m_ref = -INFINITY;   // reference maximum (scaled, log2 domain) used for the exponentials
    float l_part = 0.f;        // sum of this thread's exponentials
    bool ok = n_kv > 0;
    bool group_ok = true;      // false once the group has left the loop together after a failed wait
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      // a thread whose wait failed keeps coming to the group barrier (with good = false), so that the
      // four warps leave together and nobody is left waiting at it
      const bool good = __all_sync(full, ok && mbar_wait(&s_full[s], (j >> 1) & 1u, abort_flag, p.status,
                                                         ST_TIMEOUT_TMEM_FULL));
      const int key0 = j * FA_BN;
      // warp-uniform: does any row of this tile need masking?
      const bool tile_mask = (p.causal && key0 + FA_BN - 1 > q_off + q0) || (key0 + FA_BN > p.skv);
      uint32_t v[32];
      if (good) {
        tc_fence_after();
        tmem_ld_32x32(tmem_s + s * FA_BN + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (tile_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c * 32 + i;
            if ((p.causal && key > qpos) || key >= p.skv) v[i] = 0xff800000u;   // -inf
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          mx4[0] = fmax3(mx4[0], __uint_as_float(v[i + 0]), __uint_as_float(v[i + 1]));
          mx4[1] = fmax3(mx4[1], __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
          mx4[2] = fmax3(mx4[2], __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
          mx4[3] = fmax3(mx4[3], __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
        }
        const float mloc = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // slot j & 1: a thread can be one barrier ahead of the slowest reader of its group, never two
        tmem_st_32x32_x1(tmem_x + lane_addr + (j & 1) * 4 + c, __float_as_uint(mloc));
        tmem_st_wait();
        tc_fence_before();
      }
      if (!bar128_all(group_bar, good)) { ok = false; group_ok = false; break; }
      tc_fence_after();
      uint32_t m4[4];
      tmem_ld_32x32_x4(tmem_x + lane_addr + (j & 1) * 4, m4);
      tmem_ld_wait();
      // S has been read: its buffer may take the scores of tile j+2
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      const float mx = fmaxf(fmaxf(__uint_as_float(m4[0]), __uint_as_float(m4[1])),
                             fmaxf(__uint_as_float(m4[2]), __uint_as_float(m4[3]))) * p.scale_log2;
      float rescale = 1.f;
      bool do_rescale = false;
      if (mx > m_ref + 8.f) {       // also true on the first tile (m_ref = -inf)
        if (j > 0 && m_ref != -INFINITY) {
          rescale = fast_exp2(m_ref - mx);
          do_rescale = true;
        }
        m_ref = mx;
      }
      const float mref = (m_ref == -INFINITY) ? 0.f : m_ref;
      // O may only be touched once the previous P·V has retired (rare path: the running maximum
      // moved by more than 2^8); the decision is made warp-uniform for the .aligned TMEM accesses.
      // This thread rescales its 32 columns of O.
      if (__any_sync(full, do_rescale)) {
        const bool got = __all_sync(full, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_flag, p.status,
                                                    ST_TIMEOUT_TMEM_FULL));
        if (got) {
          tc_fence_after();
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * rescale);
          tmem_st_32x32(tmem_o + lane_addr + c * 32, o);
          tmem_st_wait();
        } else {
          ok = false;
        }
      }
      // the P buffer of this parity was last read by the P·V of tile j-2
      if (ok && j >= 2) {
        if (!__all_sync(full, mbar_wait(&pv_done[s], ((j >> 1) & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)))
          ok = false;
      }
      if (!ok) continue;            // the group learns of it at its next barrier
      // ---- P = exp2(S·scale − m), partial row sum, bf16 pack into the swizzled operand layout
      // (16-byte unit u of row r goes to unit (u ^ (r & 7)) of that row inside its 64-key chunk)
      uint8_t* p_row = smem + FaSmem::P_OFF + s * FA_TILE_BYTES + (c >> 1) * FA_CHUNK + row * 128;
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-mref, -mref);
      float2 ps2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t w[4];
#pragma unroll
        for (int h2 = 0; h2 < 4; ++h2) {
          const int i = 8 * u + 2 * h2;
          float2 x = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2);
          x.x = fast_exp2(x.x);
          x.y = fast_exp2(x.y);
          ps2[h2 & 1] = __fadd2_rn(ps2[h2 & 1], x);
          w[h2] = pack_bf16x2(x.x, x.y);
        }
        const int unit = (c & 1) * 4 + u;              // 16-byte unit inside the 64-key chunk
        *reinterpret_cast<uint4*>(p_row + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_part = l_part * rescale + (ps2[0].x + ps2[0].y) + (ps2[1].x + ps2[1].y);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    // ---- epilogue: O / l → global, LSE; this thread writes its 32 columns of the row
    const int qrow = q0 + row;
    if (n_kv > 0) {
      if (group_ok) {
        const bool good = __all_sync(full, ok && mbar_wait(&pv_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1u, abort_flag,
                                                           p.status, ST_TIMEOUT_TMEM_FULL));
        if (good) {
          tmem_st_32x32_x1(tmem_x + lane_addr + 8 + c, __float_as_uint(l_part));
          tmem_st_wait();
          tc_fence_before();
        }
        if (bar128_all(group_bar, good)) {
          tc_fence_after();
          uint32_t l4[4];
          tmem_ld_32x32_x4(tmem_x + lane_addr + 8, l4);
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, o);
          tmem_ld_wait();
          const float l_sum = (__uint_as_float(l4[0]) + __uint_as_float(l4[1])) +
                              (__uint_as_float(l4[2]) + __uint_as_float(l4[3]));
          const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
          if (qrow < p.sq) {
            __nv_bfloat16* orow = p.out + ((static_cast<size_t>(qrow) * p.b + batch) * p.hq + head) * FA_D + c * 32;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[8 * u + 0]) * inv, __uint_as_float(o[8 * u + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(o[8 * u + 2]) * inv, __uint_as_float(o[8 * u + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(o[8 * u + 4]) * inv, __uint_as_float(o[8 * u + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(o[8 * u + 6]) * inv, __uint_as_float(o[8 * u + 7]) * inv);
              reinterpret_cast<uint4*>(orow)[u] = w;
            }
            if (c == 0)
              p.lse[(static_cast<size_t>(batch) * p.hq + head) * p.sq + qrow] =
                  (l_sum > 0.f) ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
          }
        }
      }
    } else {
      // no visible key at all (only possible with a negative q_offset): zero output
      if (qrow < p.sq) {
        __nv_bfloat16* orow = p.out + ((static_cast<size_t>(qrow) * p.b + batch) * p.hq + head) * FA_D + c * 32;
        for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
        if (c == 0) p.lse[(static_cast<size_t>(batch) * p.hq + head) * p.sq + qrow] = -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace kb

namespace kb {

static int make_q_map(CUtensorMap* m, const void* q, int d, int rep, int g, int b, int sq, long qs_s, long qs_b,
                      long qs_g, long qs_r) {
  uint64_t dims[5] = {(uint64_t)d, (uint64_t)rep, (uint64_t)g, (uint64_t)b, (uint64_t)sq};
  uint64_t str[4] = {(uint64_t)qs_r * 2, (uint64_t)qs_g * 2, (uint64_t)qs_b * 2, (uint64_t)qs_s * 2};
  uint32_t box[5] = {64, 1, 1, 1, FA_BM};
  // a size-1 dimension may carry any stride; TMA still wants it to be a multiple of 16 bytes
  for (int i = 0; i < 4; ++i) if (str[i] == 0 || (str[i] & 15)) str[i] = (uint64_t)d * 2;
  return make_tmap(m, q, 2, 5, dims, str, box, 3);
}

static int make_kv_map(CUtensorMap* m, const void* ptr, int d, int g, int b, int rows, long s_s, long s_b, long s_g) {
  uint64_t dims[4] = {(uint64_t)d, (uint64_t)g, (uint64_t)b, (uint64_t)rows};
  uint32_t box[4] = {64, 1, 1, FA_BN};
  uint64_t str[3] = {(uint64_t)s_g * 2, (uint64_t)s_b * 2, (uint64_t)s_s * 2};
  for (int i = 0; i < 3; ++i) if (str[i] == 0 || (str[i] & 15)) str[i] = (uint64_t)d * 2;
  return make_tmap(m, ptr, 2, 4, dims, str, box, 3);
}

static int launch_fwd(const CUtensorMap& tmQ, const KvMaps& kv, const ChunkGeom& geom, void* out, float* lse, int sq,
                      int skv, int b, int g, int rep, float scale, int causal, int q_offset, int* status,
                      cudaStream_t stream) {
  FwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.sq = sq; p.skv = skv; p.b = b; p.hq = g * rep; p.rep = rep;
  p.q_offset = q_offset;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = status;
  p.geom = geom;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaSmem::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  dim3 grid((sq + FA_BM - 1) / FA_BM, g * rep, b);
  KB_LAUNCH(flash_attn_fwd_kernel, grid, FA_THREADS, FaSmem::TOTAL, stream, tmQ, kv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}

}  // namespace kb

// q: view [sq, b, g, rep, d] (strides in elements, d contiguous); k, v: views [skv, b, g, d];
// out: [sq, b, g*rep, d] contiguous; lse: [b, g*rep, sq] fp32.
extern "C" int kb_flash_attn_fwd(const void* q, long qs_s, long qs_b, long qs_g, long qs_r, const void* k, long ks_s,
                                 long ks_b, long ks_g, const void* v, long vs_s, long vs_b, long vs_g, void* out,
                                 float* lse, int sq, int skv, int b, int g, int rep, int d, float scale, int causal,
                                 int q_offset, int* status, cudaStream_t stream) {
  using namespace kb;
  if (d != FA_D || sq <= 0 || skv <= 0) return ST_BAD_ARG;
  CUtensorMap tmQ;
  KvMaps kv;
  memset(&kv, 0, sizeof(kv));
  int rc = make_q_map(&tmQ, q, d, rep, g, b, sq, qs_s, qs_b, qs_g, qs_r);
  if (rc) return rc;
  rc = make_kv_map(&kv.k[0], k, d, g, b, skv, ks_s, ks_b, ks_g);
  if (rc) return rc;
  rc = make_kv_map(&kv.v[0], v, d, g, b, skv, vs_s, vs_b, vs_g);
  if (rc) return rc;
  ChunkGeom geom;
  memset(&geom, 0, sizeof(geom));
  return launch_fwd(tmQ, kv, geom, out, lse, sq, skv, b, g, rep, scale, causal, q_offset, status, stream);
}

// Chunked variant.  The logical key sequence is `n_chunks` chunks of `chunk_rows` keys (a multiple of
// 128); chunk c lives in source buffer kv_src[c] (0..n_src-1) starting at row kv_row_base[c].  Every
// source is a [src_rows, b, g, d] view with the strides given (the same for all sources); k_ptrs and
// v_ptrs hold their base addresses, which may be peer mappings of other GPUs' memory.  The local
// queries are `sq / q_chunk_rows` chunks whose first rows sit at absolute positions q_pos[i].
extern "C" int kb_flash_attn_fwd_chunked(const void* q, long qs_s, long qs_b, long qs_g, long qs_r,
                                         const void* const* k_ptrs, const void* const* v_ptrs, int n_src, int src_rows,
                                         long ks_s, long ks_b, long ks_g, long vs_s, long vs_b, long vs_g,
                                         const int* kv_src, const int* kv_row_base, int n_chunks, int chunk_rows,
                                         int q_chunk_rows, const int* q_pos, void* out, float* lse, int sq, int b, int g,
                                         int rep, int d, float scale, int causal, int* status, cudaStream_t stream) {
  using namespace kb;
  ChunkGeom geom;
  int rc = fill_chunk_geom(&geom, n_src, kv_src, kv_row_base, n_chunks, chunk_rows, src_rows, q_chunk_rows, q_pos, sq);
  if (rc || d != FA_D) return ST_BAD_ARG;
  CUtensorMap tmQ;
  KvMaps kv;
  memset(&kv, 0, sizeof(kv));
  rc = make_q_map(&tmQ, q, d, rep, g, b, sq, qs_s, qs_b, qs_g, qs_r);
  if (rc) return rc;
  for (int i = 0; i < n_src; ++i) {
    rc = make_kv_map(&kv.k[i], k_ptrs[i], d, g, b, src_rows, ks_s, ks_b, ks_g);
    if (rc) return rc;
    rc = make_kv_map(&kv.v[i], v_ptrs[i], d, g, b, src_rows, vs_s, vs_b, vs_g);
    if (rc) return rc;
  }
  return launch_fwd(tmQ, kv, geom, out, lse, sq, n_chunks * chunk_rows, b, g, rep, scale, causal, 0, status, stream);
}
