// Causal GQA flash-attention backward for sm_100a (head dim 128, bf16, fp32 accumulation).
//
// One CTA owns 128 keys of one (batch, query head) and walks the query tiles that can see them:
//   warp 0      TMA producer: K and V once, then per query tile Q (two buffers, one tile ahead) and dO
//   warp 1      MMA issuer (tcgen05, accumulators in TMEM):
//                 S  = Q·Kᵀ          dP = dO·Vᵀ                       (per query tile)
//                 dV += Pᵀ·dO        dK += dSᵀ·Q        dQ = dS·K      (per query tile)
//   warps 2..17 four threads per query row, 32 key columns each: P = exp2(S·c − lse) as soon as S is
//               there (dO of the tile may still be on its way), then dS = P∘(dP − δ)·scale once dP is
//               there; both as bf16 into swizzled shared memory.  Sixteen warps, four per scheduler: with
//               one warp per scheduler this arithmetic, not the tensor pipe, set the pace of the walk
//   warps 18..21 dQ from TMEM → shared memory (the dS buffer, free between the products of one tile and
//               the dS pass of the next) → TMA reduce-add into the fp32 accumulator in global memory,
//               32 columns at a time, while the next tile is worked on
// The walk is a pipeline: S of tile i+1 is issued right behind the three products of tile i (its Q is
// already in shared memory), the dO buffer is refilled as soon as those products retire, and dQ of
// tile i is drained while P of tile i+1 is computed.
// P and dS are stored once ([q][key], keys contiguous) and serve as K-major operands (dQ) and, read
// through MN-major descriptors, as the transposed operands of dV and dK — no transposes anywhere.
// TMEM: S + dP|dQ (shared) + dV + dK = 512 columns.  dK/dV stay in TMEM across the whole walk and
// are added to fp32 accumulators at the end (query heads of one KV group run in different CTAs).
// Shared memory: K, V, Q x 2, dO, P, dS = 7 tiles of 32 KB.
// A second kernel converts the fp32 accumulators into the packed bf16 gradient of the QKV GEMM.
//
// Chunked keys and queries (context parallelism, see attention_chunks.h): K/V tiles may come from
// several source buffers (other GPUs' shards through their peer mappings, plain TMA loads), query
// tiles carry per-chunk absolute positions, and the bf16 conversion can scatter dK/dV chunk by chunk
// into the input buffer of a reduce-scatter.
//
// Replaces the FlashAttention-2 backward the reference calls through its wheel
// (kareus/flash_attn/flash_attn_interface.py:147-199).
#include "sm100.cuh"
#include "launch.h"
#include "host_utils.h"
#include "attention_chunks.h"
#include <string.h>

namespace kb {

constexpr int FB_T = 128;                      // tile edge (queries, keys) and head dim
constexpr int FB_TILE = FB_T * FB_T * 2;       // 32 KB bf16 tile as two 64-wide swizzled chunks
constexpr int FB_CHUNK = 16384;
constexpr int FB_SOFTMAX_WARPS = 16;             // 4 TMEM lane quarters x 4 chunks of 32 key columns
constexpr int FB_THREADS = (2 + FB_SOFTMAX_WARPS + 4) * 32;

struct BwdParams {
  const float* lse;      // [b, hq, sq]  natural log
  const float* delta;    // [b, hq, sq]  rowsum(dO ∘ O)
  float* dq_acc;         // [sq, b, hq, d]
  float* dk_acc;         // [skv, b, g, d]
  float* dv_acc;         // [skv, b, g, d]
  int sq, skv, b, hq, rep, q_offset, causal;
  float scale, scale_log2;
  int* status;
  ChunkGeom geom;
};

// Can any query of tile `qt` see key tile starting at k0?  (Suffix rule per query chunk.)
__device__ __forceinline__ bool q_tile_sees(const BwdParams& p, int qt, int k0) {
  if (!p.causal) return true;
  const int q0 = qt * FB_T;
  return p.geom.q_offset_of(q0, p.q_offset) + q0 + FB_T - 1 >= k0;
}

struct FbSmem {
  // Q_OFF: two consecutive tiles (buffer = iteration & 1)
  static constexpr int K_OFF = 0, V_OFF = FB_TILE, Q_OFF = 2 * FB_TILE, DO_OFF = 4 * FB_TILE, P_OFF = 5 * FB_TILE,
                       DS_OFF = 6 * FB_TILE, BAR_OFF = 7 * FB_TILE, TOTAL = BAR_OFF + 256 + 1024;
  static_assert(TOTAL <= 227 * 1024, "shared memory per CTA");
};

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Named barrier 1 of the four dQ warps; the second form returns whether `ok` held on all 128 threads.
__device__ __forceinline__ void drain_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool drain_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred P, Q;\n\tsetp.ne.u32 P, %1, 0;\n\tbar.red.and.pred Q, 1, 128, P;\n\tselp.u32 %0, 1, 0, Q;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(ok))
      : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ KvMaps kv,
                      const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmDQ,
                      const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FbSmem::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;      // [2] Q of iteration i is in buffer i & 1
  uint64_t* q_empty = bars + 3;     // [2] the MMAs that read that buffer have retired
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;    // the MMAs that read dO (and P, dS) of this iteration have retired
  uint64_t* s_full = bars + 7;      // S is in TMEM
  uint64_t* dp_full = bars + 8;     // dP is in TMEM
  uint64_t* pds_full = bars + 9;    // P and dS are in shared memory, S and dP have been read (one arrival per warp)
  uint64_t* dq_full = bars + 10;    // dQ (and this iteration's dV/dK updates) retired
  uint64_t* dq_empty = bars + 11;   // dQ has been read out of TMEM
  uint64_t* all_done = bars + 12;   // every MMA of the walk has retired
  uint64_t* stage_free = bars + 13; // the dQ reductions have read their staging area (the dS buffer)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;                 // key tile; tile 0 is seen by the most queries → first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int g = head / p.rep, r = head % p.rep;
  const int k0 = kt * FB_T;
  const int n_q = (p.sq + FB_T - 1) / FB_T;
  int n_it = 0;                              // query tiles that see this key tile
  for (int qt = 0; qt < n_q; ++qt) n_it += q_tile_sees(p, qt, k0) ? 1 : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, FB_SOFTMAX_WARPS);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 1);
    mbar_init(all_done, 1);
    mbar_init(stage_free, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // dQ of a tile goes where its dP was: dP has been read by then, and S of the next tile can be issued
  // while dQ is drained
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;
  const uint32_t t_dq = t_dp;

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      int src, srow;
      p.geom.locate(k0, src, srow);
      prefetch_tmap(&tmQ); prefetch_tmap(&kv.k[src]); prefetch_tmap(&kv.v[src]); prefetch_tmap(&tmDO);
      mbar_expect_tx(kv_full, 2 * FB_TILE);
      tma_load_4d(smem + FbSmem::K_OFF, &kv.k[src], kv_full, 0, g, batch, srow);
      tma_load_4d(smem + FbSmem::K_OFF + FB_CHUNK, &kv.k[src], kv_full, 64, g, batch, srow);
      tma_load_4d(smem + FbSmem::V_OFF, &kv.v[src], kv_full, 0, g, batch, srow);
      tma_load_4d(smem + FbSmem::V_OFF + FB_CHUNK, &kv.v[src], kv_full, 64, g, batch, srow);
      // per visible tile: Q(it) into buffer it & 1, then dO(it).  The buffer of Q(it) was released by the
      // products of tile it-2 and dO by those of tile it-1, so Q(it+1) goes out right behind dO(it): one
      // tile ahead of the MMAs.
      int it = 0;
      for (int qt = 0; qt < n_q; ++qt) {
        if (!q_tile_sees(p, qt, k0)) continue;
        const int qb = it & 1;
        const int q0 = qt * FB_T;
        if (!mbar_wait(&q_empty[qb], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        uint8_t* qdst = smem + FbSmem::Q_OFF + qb * FB_TILE;
        mbar_expect_tx(&q_full[qb], FB_TILE);
        tma_load_5d(qdst, &tmQ, &q_full[qb], 0, r, g, batch, q0);
        tma_load_5d(qdst + FB_CHUNK, &tmQ, &q_full[qb], 64, r, g, batch, q0);
        if (!mbar_wait(do_empty, (it & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(do_full, FB_TILE);
        tma_load_4d(smem + FbSmem::DO_OFF, &tmDO, do_full, 0, head, batch, q0);
        tma_load_4d(smem + FbSmem::DO_OFF + FB_CHUNK, &tmDO, do_full, 64, head, batch, q0);
        ++it;
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t id_kk = make_idesc_bf16(FB_T, FB_T, false, false);   // A K-major, B K-major
    constexpr uint32_t id_mm = make_idesc_bf16(FB_T, FB_T, true, true);     // A MN-major, B MN-major
    constexpr uint32_t id_km = make_idesc_bf16(FB_T, FB_T, false, true);    // A K-major, B MN-major
    const uint32_t a_k = smem_u32(smem + FbSmem::K_OFF), a_v = smem_u32(smem + FbSmem::V_OFF);
    const uint32_t a_q0 = smem_u32(smem + FbSmem::Q_OFF), a_do = smem_u32(smem + FbSmem::DO_OFF);
    const uint32_t a_p = smem_u32(smem + FbSmem::P_OFF), a_ds = smem_u32(smem + FbSmem::DS_OFF);
    auto kmaj = [](uint32_t base, int k) { return make_smem_desc(base + (k >> 2) * FB_CHUNK + (k & 3) * 32, 16, 1024); };
    auto mnmaj = [](uint32_t base, int k) { return make_smem_desc(base + k * 2048, FB_CHUNK, 1024); };
    bool ok = n_it > 0;
    if (ok) ok = mbar_wait(kv_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL);
    if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, p.status, ST_TIMEOUT_FULL);
    if (ok) {
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(t_s, kmaj(a_q0, k), kmaj(a_k, k), id_kk, k > 0);
        umma_commit(s_full);
      }
      __syncwarp();
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const uint32_t ph = it & 1u;
      const uint32_t a_q = a_q0 + (it & 1) * FB_TILE;
      // dP(it) overwrites the columns that held dQ(it-1)
      if (!mbar_wait(do_full, ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
      if (!mbar_wait(dq_empty, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(t_dp, kmaj(a_do, k), kmaj(a_v, k), id_kk, k > 0);
        umma_commit(dp_full);
      }
      __syncwarp();
      if (!mbar_wait(pds_full, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(t_dv, mnmaj(a_p, k), mnmaj(a_do, k), id_mm, (it > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(t_dk, mnmaj(a_ds, k), mnmaj(a_q, k), id_mm, (it > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(t_dq, kmaj(a_ds, k), mnmaj(a_k, k), id_km, k > 0);
        umma_commit(&q_empty[it & 1]);
        umma_commit(do_empty);
        umma_commit(dq_full);
      }
      __syncwarp();
      if (it + 1 < n_it) {
        // S of the next tile: its Q is already there, and S(it) has been read (pds_full above)
        const int nb = (it + 1) & 1;
        if (!mbar_wait(&q_full[nb], ((it + 1) >> 1) & 1u, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_qn = a_q0 + nb * FB_TILE;
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ss(t_s, kmaj(a_qn, k), kmaj(a_k, k), id_kk, k > 0);
          umma_commit(s_full);
        }
        __syncwarp();
      }
    }
    if (ok && lane == 0) umma_commit(all_done);
    __syncwarp();
  } else {
    const int quarter = warp & 3;            // TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool softmax_role = warp < 2 + FB_SOFTMAX_WARPS;
    const int c = (warp - 2) >> 2;           // softmax warps: chunk of 32 key columns
    bool ok = n_it > 0;
    int it = -1;
    if (softmax_role) {
      const float lg2e = 1.4426950408889634f;
      // 16-byte units of this thread inside its row of P / dS (two 64-wide swizzled chunks per row)
      uint32_t unit_off[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        unit_off[u] = (c >> 1) * FB_CHUNK + row * 128 + ((((c & 1) * 4 + u) ^ (row & 7)) << 4);
      for (int qt = 0; qt < n_q && ok; ++qt) {
        if (!q_tile_sees(p, qt, k0)) continue;
        ++it;
        const uint32_t ph = it & 1u;
        const int q0 = qt * FB_T;
        const int q_off = p.geom.q_offset_of(q0, p.q_offset);
        const int qrow = q0 + row;
        const int qpos = q_off + qrow;
        const bool valid = qrow < p.sq;
        const size_t stat = (static_cast<size_t>(batch) * p.hq + head) * p.sq + (valid ? qrow : 0);
        const float lse2 = valid ? p.lse[stat] * lg2e : 0.f;
        const float dlt = valid ? p.delta[stat] : 0.f;
        const bool tile_mask = (p.causal && k0 + FB_T - 1 > q_off + q0) || (k0 + FB_T > p.skv) || (q0 + FB_T > p.sq);
        // S(it) ready: the products of tile it-1 were issued before it, so P and dS buffers are free
        if (!mbar_wait(s_full, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        uint32_t pk[16];                       // this thread's 32 values of P as packed bf16, kept for dS
        {
          uint32_t sv[32];
          tmem_ld_32x32(t_s + lane_addr + c * 32, sv);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int h2 = 0; h2 < 4; ++h2) {
              const int i = 8 * u + 2 * h2;
              float e0 = bwd_exp2(__uint_as_float(sv[i]) * p.scale_log2 - lse2);
              float e1 = bwd_exp2(__uint_as_float(sv[i + 1]) * p.scale_log2 - lse2);
              if (tile_mask) {
                const int key = k0 + c * 32 + i;
                if (!valid || (p.causal && key > qpos) || key >= p.skv) e0 = 0.f;
                if (!valid || (p.causal && key + 1 > qpos) || key + 1 >= p.skv) e1 = 0.f;
              }
              pk[u * 4 + h2] = pack_bf16x2(e0, e1);
            }
            *reinterpret_cast<uint4*>(smem + FbSmem::P_OFF + unit_off[u]) =
                make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
          }
        }
        if (!mbar_wait(dp_full, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        // the dS buffer doubled as staging area of the previous tile's dQ reductions
        if (it > 0 && !mbar_wait(stage_free, (it - 1) & 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t dv[32];
          tmem_ld_32x32(t_dp + lane_addr + c * 32, dv);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t wd[4];
#pragma unroll
            for (int h2 = 0; h2 < 4; ++h2) {
              const int i = 8 * u + 2 * h2;
              const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[u * 4 + h2]));
              const float d0 = e.x * (__uint_as_float(dv[i]) - dlt) * p.scale;
              const float d1 = e.y * (__uint_as_float(dv[i + 1]) - dlt) * p.scale;
              wd[h2] = pack_bf16x2(d0, d1);
            }
            *reinterpret_cast<uint4*>(smem + FbSmem::DS_OFF + unit_off[u]) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_full);
      }
    } else {
      // dQ tile → fp32 reductions into the global accumulator, 32 columns (16 KB) at a time through the two
      // halves of the dS buffer: 128-byte rows with their 16-byte units swizzled by row, as the tensor
      // map of the accumulator expects
      const bool leader = threadIdx.x == (2 + FB_SOFTMAX_WARPS) * 32;
      uint8_t* stage = smem + FbSmem::DS_OFF;
      for (int qt = 0; qt < n_q && ok; ++qt) {
        if (!q_tile_sees(p, qt, k0)) continue;
        ++it;
        const uint32_t ph = it & 1u;
        // one decision for the 128 threads (they meet at named barriers below); the leader comes here only
        // after the previous tile's reductions have read the staging area
        ok = drain_all(mbar_wait(dq_full, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint8_t* buf = stage + (cc & 1) * 16384;
          if (cc >= 2) {
            if (leader) tma_store_wait_read<1>();      // the reduction of chunk cc-2 has read this half
            drain_sync();
          }
          uint32_t v[32];
          tmem_ld_32x32(t_dq + lane_addr + cc * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(buf + row * 128 + ((j ^ (row & 7)) << 4)) =
                make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          if (cc == 3) tc_fence_before();
          drain_sync();
          if (leader) {
            tma_reduce_add_4d(&tmDQ, buf, cc * 32, head, batch, qt * FB_T);   // rows past sq are clipped
            tma_store_commit();
          }
        }
        if (leader) {
          mbar_arrive(dq_empty);                       // every thread's TMEM reads preceded the last barrier
          tma_store_wait_read<0>();
          mbar_arrive(stage_free);
        }
      }
      if (leader) tma_store_wait<0>();                 // nothing in flight out of shared memory at exit
    }
    // dV and dK of this key tile → fp32 accumulators (rows = keys); softmax warp (quarter, c) takes
    // columns 32c..32c+31 of both
    if (n_it > 0 && softmax_role) {
      if (ok) ok = mbar_wait(all_done, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const int key = k0 + row;
      const bool kvalid = ok && key < p.skv;
      const size_t base = ((static_cast<size_t>(kvalid ? key : 0) * p.b + batch) * (p.hq / p.rep) + g) * FB_T;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        float* dst = (which == 0 ? p.dv_acc : p.dk_acc) + base + c * 32;
        uint32_t v[32];
        tmem_ld_32x32((which == 0 ? t_dv : t_dk) + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (kvalid) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            red_add_v4(dst + 4 * j, __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
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

// delta[b, h, s] = Σ_d dO[s,b,h,d] · O[s,b,h,d]   (both [s,b,h,d] contiguous), one warp per row
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                  float* __restrict__ delta, int S, int B, int H) {
  const long rows = static_cast<long>(S) * B * H;
  const int lane = threadIdx.x & 31;
  for (long w = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < rows;
       w += (static_cast<long>(gridDim.x) * blockDim.x) >> 5) {
    const uint2 a = reinterpret_cast<const uint2*>(dO + w * FB_T)[lane];
    const uint2 b = reinterpret_cast<const uint2*>(O + w * FB_T)[lane];
    const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
    float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
      const int h = static_cast<int>(w % H);
      const long sb = w / H;
      const int bb = static_cast<int>(sb % B);
      const long ss = sb / B;
      delta[(static_cast<long>(bb) * H + h) * S + ss] = s;
    }
  }
}

// fp32 accumulator [rows(s,b), heads, d] → bf16 strided view (strides in elements per s, b, head)
__global__ void attn_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long n_vec, int B,
                                    int G, int R, long st_s, long st_b, long st_g, long st_r) {
  // one thread per 4 elements of d
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int dv = static_cast<int>(i % (FB_T / 4));
    long rest = i / (FB_T / 4);
    const int rr = static_cast<int>(rest % R); rest /= R;
    const int gg = static_cast<int>(rest % G); rest /= G;
    const int bb = static_cast<int>(rest % B);
    const long ss = rest / B;
    const float4 v = reinterpret_cast<const float4*>(acc)[i];
    __nv_bfloat16* o = out + ss * st_s + bb * st_b + gg * st_g + rr * st_r + dv * 4;
    uint2 w;
    *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(o) = w;
  }
}

static int make_qkv_map(CUtensorMap* m, const void* ptr, int d, int inner_heads, int g, int b, int s, long st_r,
                        long st_g, long st_b, long st_s, int rank5) {
  if (rank5) {
    uint64_t dims[5] = {(uint64_t)d, (uint64_t)inner_heads, (uint64_t)g, (uint64_t)b, (uint64_t)s};
    uint64_t str[4] = {(uint64_t)st_r * 2, (uint64_t)st_g * 2, (uint64_t)st_b * 2, (uint64_t)st_s * 2};
    uint32_t box[5] = {64, 1, 1, 1, FB_T};
    for (int i = 0; i < 4; ++i) if (str[i] == 0 || (str[i] & 15)) str[i] = (uint64_t)d * 2;
    return make_tmap(m, ptr, 2, 5, dims, str, box, 3);
  }
  uint64_t dims[4] = {(uint64_t)d, (uint64_t)g, (uint64_t)b, (uint64_t)s};
  uint64_t str[3] = {(uint64_t)st_g * 2, (uint64_t)st_b * 2, (uint64_t)st_s * 2};
  uint32_t box[4] = {64, 1, 1, FB_T};
  for (int i = 0; i < 3; ++i) if (str[i] == 0 || (str[i] & 15)) str[i] = (uint64_t)d * 2;
  return make_tmap(m, ptr, 2, 4, dims, str, box, 3);
}

}  // namespace kb

using namespace kb;

// Scratch: `work` must hold (sq*b*hq*d + 2*skv*b*g*d + b*hq*sq) floats; it is zeroed here.
extern "C" long kb_flash_attn_bwd_scratch_floats(int sq, int skv, int b, int g, int rep, int d) {
  return (long)sq * b * g * rep * d + 2L * skv * b * g * d + (long)b * g * rep * sq;
}

namespace kb {

struct RowMap {
  int chunk_rows;                    // 0: rows map to themselves
  int base[MAX_KV_CHUNKS];
};

// fp32 accumulator [logical rows, b, g, d] → bf16 rows of a strided destination where logical chunk c
// starts at destination row map.base[c] (dK/dV straight into the layout a reduce-scatter expects)
__global__ void attn_convert_chunked_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long n_vec,
                                            int B, int G, long st_s, long st_b, long st_g, RowMap map) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int dv = static_cast<int>(i % (FB_T / 4));
    long rest = i / (FB_T / 4);
    const int gg = static_cast<int>(rest % G); rest /= G;
    const int bb = static_cast<int>(rest % B);
    long ss = rest / B;
    if (map.chunk_rows > 0) {
      const int c = static_cast<int>(ss / map.chunk_rows);
      ss = map.base[c] + (ss - static_cast<long>(c) * map.chunk_rows);
    }
    const float4 v = reinterpret_cast<const float4*>(acc)[i];
    __nv_bfloat16* o = out + ss * st_s + bb * st_b + gg * st_g + dv * 4;
    uint2 w;
    *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(o) = w;
  }
}

struct BwdOut {
  void* dq; long dqs_s, dqs_b, dqs_g, dqs_r;
  void* dk; long dks_s, dks_b, dks_g;
  void* dv; long dvs_s, dvs_b, dvs_g;
  RowMap dk_rows, dv_rows;
};

static int launch_bwd(const CUtensorMap& tmQ, const KvMaps& kv, const ChunkGeom& geom, const void* o, const void* dO,
                      const float* lse, const BwdOut& out, float* work, int sq, int skv, int b, int g, int rep, int d,
                      float scale, int causal, int q_offset, int last_key, int* status, cudaStream_t stream) {
  const int hq = g * rep;
  const long n_dq = (long)sq * b * hq * d, n_dkv = (long)skv * b * g * d;
  float* dq_acc = work;
  float* dk_acc = dq_acc + n_dq;
  float* dv_acc = dk_acc + n_dkv;
  float* delta = dv_acc + n_dkv;
  cudaError_t e = kb::memset_async(work, 0, sizeof(float) * (n_dq + 2 * n_dkv), stream);
  if (e != cudaSuccess) return 1000 + (int)e;
  {
    const long rows = (long)sq * b * hq;
    long blocks = (rows * 32 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    KB_LAUNCH(attn_delta_kernel, (int)blocks, 256, 0, stream, (const __nv_bfloat16*)dO, (const __nv_bfloat16*)o, delta, sq, b, hq);
  }
  CUtensorMap tmDO;
  int rc = make_qkv_map(&tmDO, dO, d, 1, hq, b, sq, 0, d, (long)hq * d, (long)b * hq * d, 0);
  if (rc) return rc;
  BwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc; p.dk_acc = dk_acc; p.dv_acc = dv_acc;
  p.sq = sq; p.skv = skv; p.b = b; p.hq = hq; p.rep = rep; p.q_offset = q_offset; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.geom = geom;
  static bool configured = false;
  if (!configured) {
    e = cudaFuncSetAttribute(flash_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSmem::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  CUtensorMap tmDQ;
  {
    // fp32 accumulator [sq, b, hq, d]: boxes of 128 rows x 32 columns (128 bytes, swizzled) of one (b, head)
    uint64_t dims[4] = {(uint64_t)d, (uint64_t)hq, (uint64_t)b, (uint64_t)sq};
    uint64_t str[3] = {(uint64_t)d * 4, (uint64_t)hq * d * 4, (uint64_t)b * hq * d * 4};
    uint32_t box[4] = {32, 1, 1, FB_T};
    rc = make_tmap(&tmDQ, dq_acc, 4, 4, dims, str, box, 3);
    if (rc) return rc;
  }
  int n_kv = (skv + FB_T - 1) / FB_T;
  if (causal) {
    const int lim = (last_key + FB_T - 1) / FB_T;      // keys >= last_key are seen by no query
    if (lim < n_kv) n_kv = lim > 0 ? lim : 0;
  }
  if (n_kv > 0) {
    dim3 grid(n_kv, hq, b);
    KB_LAUNCH(flash_attn_bwd_kernel, grid, FB_THREADS, FbSmem::TOTAL, stream, tmQ, kv, tmDO, tmDQ, p);
  }
  {
    long nvec = n_dq / 4;
    long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    KB_LAUNCH(attn_convert_kernel, (int)blocks, 256, 0, stream, (const float*)dq_acc, (__nv_bfloat16*)out.dq, nvec, b, g, rep,
              out.dqs_s, out.dqs_b, out.dqs_g, out.dqs_r);
    nvec = n_dkv / 4;
    blocks = (nvec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    KB_LAUNCH(attn_convert_chunked_kernel, (int)blocks, 256, 0, stream, (const float*)dk_acc, (__nv_bfloat16*)out.dk, nvec, b,
              g, out.dks_s, out.dks_b, out.dks_g, out.dk_rows);
    KB_LAUNCH(attn_convert_chunked_kernel, (int)blocks, 256, 0, stream, (const float*)dv_acc, (__nv_bfloat16*)out.dv, nvec, b,
              g, out.dvs_s, out.dvs_b, out.dvs_g, out.dv_rows);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}

}  // namespace kb

// q: view [sq,b,g,rep,d]; k,v: views [skv,b,g,d]; o, dO: [sq,b,hq,d] contiguous; lse [b,hq,sq].
// dq/dk/dv: destination views with the same geometry as q/k/v (strides in elements).
extern "C" int kb_flash_attn_bwd(const void* q, long qs_s, long qs_b, long qs_g, long qs_r, const void* k, long ks_s,
                                 long ks_b, long ks_g, const void* v, long vs_s, long vs_b, long vs_g, const void* o,
                                 const void* dO, const float* lse, void* dq, long dqs_s, long dqs_b, long dqs_g,
                                 long dqs_r, void* dk, long dks_s, long dks_b, long dks_g, void* dv, long dvs_s,
                                 long dvs_b, long dvs_g, float* work, int sq, int skv, int b, int g, int rep, int d,
                                 float scale, int causal, int q_offset, int* status, cudaStream_t stream) {
  if (d != FB_T || sq <= 0 || skv <= 0) return ST_BAD_ARG;
  CUtensorMap tmQ;
  KvMaps kv;
  memset(&kv, 0, sizeof(kv));
  int rc = make_qkv_map(&tmQ, q, d, rep, g, b, sq, qs_r, qs_g, qs_b, qs_s, 1);
  if (rc) return rc;
  rc = make_qkv_map(&kv.k[0], k, d, 1, g, b, skv, 0, ks_g, ks_b, ks_s, 0);
  if (rc) return rc;
  rc = make_qkv_map(&kv.v[0], v, d, 1, g, b, skv, 0, vs_g, vs_b, vs_s, 0);
  if (rc) return rc;
  ChunkGeom geom;
  memset(&geom, 0, sizeof(geom));
  BwdOut out;
  memset(&out, 0, sizeof(out));
  out.dq = dq; out.dqs_s = dqs_s; out.dqs_b = dqs_b; out.dqs_g = dqs_g; out.dqs_r = dqs_r;
  out.dk = dk; out.dks_s = dks_s; out.dks_b = dks_b; out.dks_g = dks_g;
  out.dv = dv; out.dvs_s = dvs_s; out.dvs_b = dvs_b; out.dvs_g = dvs_g;
  return launch_bwd(tmQ, kv, geom, o, dO, lse, out, work, sq, skv, b, g, rep, d, scale, causal, q_offset,
                    q_offset + sq, status, stream);
}

// Chunked variant (see kb_flash_attn_fwd_chunked for the key/query chunk description).  dK and dV of the
// whole logical key range go to ONE destination `dkv` ([rows, b, g, d] with the strides given): logical
// chunk c of dK starts at row dk_row_base[c], of dV at dv_row_base[c] — e.g. the rank-ordered input
// buffer of a reduce-scatter, so that nothing is copied between this kernel and the collective.
extern "C" int kb_flash_attn_bwd_chunked(const void* q, long qs_s, long qs_b, long qs_g, long qs_r,
                                         const void* const* k_ptrs, const void* const* v_ptrs, int n_src, int src_rows,
                                         long ks_s, long ks_b, long ks_g, long vs_s, long vs_b, long vs_g,
                                         const int* kv_src, const int* kv_row_base, int n_chunks, int chunk_rows,
                                         int q_chunk_rows, const int* q_pos, const void* o, const void* dO,
                                         const float* lse, void* dq, long dqs_s, long dqs_b, long dqs_g, long dqs_r,
                                         void* dkv, long dkvs_s, long dkvs_b, long dkvs_g, const int* dk_row_base,
                                         const int* dv_row_base, float* work, int sq, int b, int g, int rep, int d,
                                         float scale, int causal, int* status, cudaStream_t stream) {
  ChunkGeom geom;
  int rc = fill_chunk_geom(&geom, n_src, kv_src, kv_row_base, n_chunks, chunk_rows, src_rows, q_chunk_rows, q_pos, sq);
  if (rc || d != FB_T) return ST_BAD_ARG;
  const int skv = n_chunks * chunk_rows;
  CUtensorMap tmQ;
  KvMaps kv;
  memset(&kv, 0, sizeof(kv));
  rc = make_qkv_map(&tmQ, q, d, rep, g, b, sq, qs_r, qs_g, qs_b, qs_s, 1);
  if (rc) return rc;
  for (int i = 0; i < n_src; ++i) {
    rc = make_qkv_map(&kv.k[i], k_ptrs[i], d, 1, g, b, src_rows, 0, ks_g, ks_b, ks_s, 0);
    if (rc) return rc;
    rc = make_qkv_map(&kv.v[i], v_ptrs[i], d, 1, g, b, src_rows, 0, vs_g, vs_b, vs_s, 0);
    if (rc) return rc;
  }
  BwdOut out;
  memset(&out, 0, sizeof(out));
  out.dq = dq; out.dqs_s = dqs_s; out.dqs_b = dqs_b; out.dqs_g = dqs_g; out.dqs_r = dqs_r;
  out.dk = dkv; out.dks_s = dkvs_s; out.dks_b = dkvs_b; out.dks_g = dkvs_g;
  out.dv = dkv; out.dvs_s = dkvs_s; out.dvs_b = dkvs_b; out.dvs_g = dkvs_g;
  out.dk_rows.chunk_rows = out.dv_rows.chunk_rows = chunk_rows;
  int last_key = 0;
  for (int i = 0; i < sq / q_chunk_rows; ++i) last_key = q_pos[i] + q_chunk_rows > last_key ? q_pos[i] + q_chunk_rows : last_key;
  for (int c = 0; c < n_chunks; ++c) {
    out.dk_rows.base[c] = dk_row_base[c];
    out.dv_rows.base[c] = dv_row_base[c];
  }
  return launch_bwd(tmQ, kv, geom, o, dO, lse, out, work, sq, skv, b, g, rep, d, scale, causal, 0, last_key, status,
                    stream);
}
