// Tensor-parallel GEMMs fused with their sequence-parallel collective (sm_100a, bf16):
//
//   ag_gemm:  Y[M,N] = AllGather_rows(X_shard)[M,K] · W[N,K]ᵀ      (QKV, FC1 forward)
//   gemm_rs:  Y_shard[M/tp,N] = ReduceScatter_rows(A[M,K] · W[N,K]ᵀ) (out-proj, FC2 forward)
//
// One kernel does the math and moves the collective's bytes over NVLink, tile by tile:
//
// * ag_gemm — CTAs 0..n_comm-1 are copy drivers: one thread per CTA streams the peers' shards with
//   bulk asynchronous copies (peer global → shared-memory ring → local gathered buffer) and, after
//   every 128-row tile, publishes a per-tile flag.  The remaining CTAs run the tcgen05 GEMM; they
//   visit row tiles in arrival order (own shard first, then rank+1, rank+2, …) and the TMA producer
//   waits for a tile's flag only if the tile is remote.  No tile crosses NVLink more than once, no
//   TMA multicast is used, and the gathered activations stay in the buffer for the wgrad GEMM.
// * gemm_rs — the GEMM CTAs visit row tiles in owner order (rank+1 first, own rows last).  For a
//   peer's rows the epilogue sends the bf16 partial tile straight into the owner's staging slot (TMA
//   stores out of a double-buffered shared-memory staging area through per-peer tensor maps; with
//   KAREUS_RS_TMA=0 plain 128-byte row-segment stores) and bumps a per-tile counter there.  For
//   its own rows the epilogue waits for the other ranks' counters of that tile, adds their staged
//   partials in fp32 and writes the finished sequence shard: no separate reduction pass exists.
//   One extra CTA runs the start barrier (peers must have entered the call before their staging is
//   written).
//
// The plan's `sm_num` knob ("SMs given to the collective") reaches both kernels as `n_comm`:
// * ag_gemm: the number of copy-driver CTAs (more drivers pull the peers' shards faster and take SMs
//   from the GEMM role);
// * gemm_rs: the number of SMs the kernel leaves ALONE — its GEMM CTAs number num_sms − 1 − n_comm —
//   so that the other nanobatch's kernels on the compute stream keep that many SMs while this
//   link-bound kernel runs (0: use the whole budget).  There are no separate reducer CTAs: the sums
//   are finished in the own-row epilogues.
//
// Switch-multicast variants (kb_ag_gemm_mc_bf16 / kb_gemm_rs_mc_bf16; buffers inside an NVLS buffer,
// parallel/nvls.py).  The SMs then touch NVLink far less:
// * ag_gemm: the drivers PUSH this rank's own shard once with multimem.st; the switch replicates it
//   into all ranks' gathered buffers (posted writes, 1/7 of the bytes per sending SM) and a
//   multimem.red bumps the tile's ready flag everywhere.
// * gemm_rs: every partial tile is stored to LOCAL staging (the epilogue runs at plain-GEMM speed, the
//   release that precedes the tile counter covers local writes only), and the owner fetches each of
//   its tiles already summed over all ranks with multimem.ld_reduce.
// Every wait is bounded (status word + return).  Role of the reference's separate cuBLASLt GEMM followed
// or preceded by an all-reduce kernel (kareus/megatron/core/extensions/ops/te_linear.py:303-445,
// 3rdparty/mscclpp/python/mscclpp_benchmark/allreduce.cu:155-246).
#include "sm100.cuh"
#include "launch.h"
#include "peer.cuh"
#include "host_utils.h"
#include <stdlib.h>
#include <string.h>

namespace kb {

constexpr int FG_BM = 128;
constexpr int FG_BK = 64;
constexpr int FG_STAGES = 4;
constexpr int FG_THREADS = 192;
constexpr int FG_CHUNK = 32768;      // bytes per bulk copy of a copy driver
constexpr int FG_SLOTS = 6;          // copy ring depth (6 x 32 KB)

enum { MODE_AG = 1, MODE_RS = 2 };

struct FusedParams {
  PeerCtx peer;
  int mode;
  int n_first;            // AG: copy-driver CTAs in front of the GEMM CTAs
  int n_gemm;             // GEMM CTAs
  int n_last;             // RS: reducer CTAs behind the GEMM CTAs
  int rows_per_rank;      // Ms
  uint32_t epoch;
  // AG
  uint64_t xg_off;        // gathered buffer [M, K] in every heap
  uint32_t* ready;        // local flags, one per 128-row tile of the gathered buffer
  // RS
  uint64_t stage_off;     // staging [world][Ms][N] in every heap
  uint64_t cnt_off;       // counters [world][Ms/128][tiles_n] (uint32) in every heap
  uint32_t* go;           // local flag: peers have entered this call
  __nv_bfloat16* out;     // [Ms, N]
  // switch-multicast variants: local and multicast view of the NVLS buffer (null: peer loads/stores);
  // xg_off / stage_off / ready_off are then offsets inside that buffer
  uint8_t* uc;
  uint8_t* mc;
  uint64_t ready_off;     // AG: uint32 per 128-row tile, bumped on every rank by the tile's sender
  int push_tma;           // RS over peer memory: partial tiles leave through TMA stores (maps in StageMaps)
  // AG: gathered buffer [M, K] in ordinary local memory (null: inside the heap at xg_off).  xg_off then names
  // the [Ms, K] buffer that holds each rank's own shard in its heap; the caller has also put this rank's
  // shard into its rows of xg_local.
  uint8_t* xg_local;
};

// RS: one tensor map per peer over this rank's slot [rows_per_rank, N] of that peer's staging area.  The
// epilogue hands each 32-row x 64-column block to the TMA unit instead of storing it with the warp's lanes:
// the copy engine of the SM keeps far more bytes in flight towards the peer than 128 storing threads do.
struct StageMaps {
  CUtensorMap m[MAX_PEERS];
};

template <int BN>
struct FgSmem {
  static constexpr int A_BYTES = FG_BM * FG_BK * 2;
  static constexpr int B_BYTES = BN * FG_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGE_BYTES * FG_STAGES;
  static constexpr int STG_BYTES = 4 * 2 * 4096;    // per epilogue warp two 4 KB staging buffers (1 KiB aligned:
                                                   // a TMA store reads them with the 128-byte swizzle)
  static constexpr int BAR_OFF = TILE_BYTES + STG_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ----------------------------------------------------------------------------- copy driver (AG)
__device__ void ag_copy_role(const FusedParams& p, int K, uint8_t* smem, uint64_t* bars, volatile int* abort_flag,
                             int* ok_slot) {
  const PeerCtx& c = p.peer;
  const int cta = blockIdx.x;
  if (!peer_barrier(c, cta, static_cast<uint64_t>(p.epoch) * 4 + 1, ok_slot)) return;
  if (threadIdx.x == 0) {
    uint64_t* full = bars;                  // [FG_SLOTS], placed behind the ring
    const long tile_bytes = static_cast<long>(FG_BM) * K * 2;
    const int tiles_per_rank = p.rows_per_rank / FG_BM;
    const int remote_tiles = tiles_per_rank * (c.world - 1);
    uint32_t issued = 0;                    // chunks loaded so far by this driver (ring position)
    bool ok = true;
    // remote tiles in arrival order: all tiles of rank+1, then rank+2, ...; drivers take them round-robin
    for (int rt = cta; rt < remote_tiles && ok; rt += p.n_first) {
      const int src = (c.rank + 1 + rt / tiles_per_rank) % c.world;
      const int tile = src * tiles_per_rank + rt % tiles_per_rank;     // tile index in the gathered buffer
      const uint8_t* from = p.xg_local ? c.base[src] + p.xg_off + (rt % tiles_per_rank) * tile_bytes
                                       : c.base[src] + p.xg_off + tile * tile_bytes;
      uint8_t* to = (p.xg_local ? p.xg_local : c.base[c.rank] + p.xg_off) + tile * tile_bytes;
      const int nchunks = static_cast<int>((tile_bytes + FG_CHUNK - 1) / FG_CHUNK);
      int loaded = 0, stored = 0;
      while (stored < nchunks && ok) {
        // keep the ring full
        // a slot is refilled only after the store that used it has read it: at most one store is still
        // reading (chunk stored-1), and chunk `loaded` shares its slot only when loaded - (stored-1) ==
        // FG_SLOTS, so loads may run FG_SLOTS-1 chunks ahead of the stores
        while (loaded < nchunks && loaded - stored < FG_SLOTS - 1) {
          const int slot = (issued + loaded) % FG_SLOTS;
          const long o = static_cast<long>(loaded) * FG_CHUNK;
          const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long>(FG_CHUNK), tile_bytes - o));
          mbar_expect_tx(&full[slot], bytes);
          bulk_g2s(smem + slot * FG_CHUNK, from + o, bytes, &full[slot]);
          ++loaded;
        }
        const int slot = (issued + stored) % FG_SLOTS;
        const uint32_t ph = ((issued + stored) / FG_SLOTS) & 1u;
        if (!mbar_wait(&full[slot], ph, abort_flag, c.status, ST_TIMEOUT_PEER)) { ok = false; break; }
        const long o = static_cast<long>(stored) * FG_CHUNK;
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long>(FG_CHUNK), tile_bytes - o));
        bulk_s2g(to + o, smem + slot * FG_CHUNK, bytes);
        tma_store_commit();
        ++stored;
        tma_store_wait_read<1>();
      }
      issued += nchunks;
      tma_store_wait<0>();                  // the tile's bytes are in local memory
      __threadfence();
      st_release_gpu_u32(&p.ready[tile], p.epoch);
    }
    tma_store_wait<0>();
  }
  // peers may still be reading this rank's shard: do not let the kernel (and the next writer of the
  // shard) get ahead of them
  peer_barrier(c, cta, static_cast<uint64_t>(p.epoch) * 4 + 2, ok_slot);
}

// ----------------------------------------------------------------------------- push driver (AG, multicast)
// This rank's own shard, tile by tile, to every rank's gathered buffer through the switch.
__device__ void ag_push_role(const FusedParams& p, int K, int* ok_slot) {
  const PeerCtx& c = p.peer;
  const int cta = blockIdx.x;
  // every rank has entered this call: the previous contents of all gathered buffers have been consumed
  if (!peer_barrier(c, cta, static_cast<uint64_t>(p.epoch) * 4 + 1, ok_slot)) return;
  const long tile_vecs = static_cast<long>(FG_BM) * K * 2 / 16;
  const int tiles_per_rank = p.rows_per_rank / FG_BM;
  for (int lt = cta; lt < tiles_per_rank; lt += p.n_first) {
    const int tile = c.rank * tiles_per_rank + lt;
    const uint4* src = reinterpret_cast<const uint4*>(p.uc + p.xg_off) + tile * tile_vecs;
    uint4* dst = reinterpret_cast<uint4*>(p.mc + p.xg_off) + tile * tile_vecs;
    long i = threadIdx.x;
    for (; i + 3 * FG_THREADS < tile_vecs; i += 4 * FG_THREADS) {
      const uint4 a = src[i], b = src[i + FG_THREADS], d = src[i + 2 * FG_THREADS], e = src[i + 3 * FG_THREADS];
      mm_st_bf16x8(dst + i, a);
      mm_st_bf16x8(dst + i + FG_THREADS, b);
      mm_st_bf16x8(dst + i + 2 * FG_THREADS, d);
      mm_st_bf16x8(dst + i + 3 * FG_THREADS, e);
    }
    for (; i < tile_vecs; i += FG_THREADS) mm_st_bf16x8(dst + i, src[i]);
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_sys();      // the tile's stores (cumulative over the CTA through the barrier) before its flag
      mm_red_add_u32(p.mc + p.ready_off + static_cast<uint64_t>(tile) * 4, 1u);
    }
  }
}

// ----------------------------------------------------------------------------- kernel
// B_MN: the weight operand is stored [K rows][N contiguous] (dgrad: dY·W with W as [N_red, K_out]).
template <int BN, bool B_MN>
__global__ void __launch_bounds__(FG_THREADS, 1)
fused_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ StageMaps stage_maps, const FusedParams p, int M, int N, int K) {
  using S = FgSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  uint64_t* empty = full + FG_STAGES;
  uint64_t* tfull = empty + FG_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* ok_slot = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + FG_BM - 1) / FG_BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int nk = (K + FG_BK - 1) / FG_BK;
  const PeerCtx& c = p.peer;
  int* status = c.status;

  // ---- non-GEMM roles
  if (static_cast<int>(blockIdx.x) < p.n_first) {
    uint64_t* ring_bars = reinterpret_cast<uint64_t*>(smem + FG_SLOTS * FG_CHUNK);
    volatile int* ring_abort = reinterpret_cast<volatile int*>(ring_bars + FG_SLOTS);
    int* ring_ok = const_cast<int*>(ring_abort) + 1;
    if (threadIdx.x == 0) {
      for (int i = 0; i < FG_SLOTS; ++i) mbar_init(&ring_bars[i], 1);
      *ring_abort = 0;
      *ring_ok = 1;
      mbar_fence_init();
    }
    __syncthreads();
    if (p.mc != nullptr) ag_push_role(p, K, ring_ok);
    else ag_copy_role(p, K, smem, ring_bars, ring_abort, ring_ok);
    return;
  }
  if (static_cast<int>(blockIdx.x) >= p.n_first + p.n_gemm) {
    if (threadIdx.x == 0) *ok_slot = 1;
    __syncthreads();
    if (static_cast<int>(blockIdx.x) == p.n_first + p.n_gemm) {
      // tell this rank's epilogues that every peer has entered the call (their staging is free)
      const bool ok = peer_barrier(c, 0, static_cast<uint64_t>(p.epoch) * 4 + 1, ok_slot);
      if (threadIdx.x == 0 && ok) st_release_gpu_u32(p.go, p.epoch);
    }
    return;
  }

  // ---- GEMM role
  const int cta = blockIdx.x - p.n_first;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  if (threadIdx.x == 0) {
    for (int i = 0; i < FG_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile t -> (row tile, column tile): rank-rotated blocks of rows, m fastest inside a block
  const int tiles_per_rank = p.rows_per_rank / FG_BM;
  const int per_owner = tiles_per_rank * tiles_n;
  auto coords = [&](int t, int& tm, int& tn) {
    const int blk = t / per_owner;
    const int owner = (c.rank + (p.mode == MODE_RS ? 1 : 0) + blk) % c.world;
    const int r = t - blk * per_owner;
    tm = owner * tiles_per_rank + r % tiles_per_rank;
    tn = r / tiles_per_rank;
  };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += p.n_gemm) {
        int tm, tn;
        coords(t, tm, tn);
        if (p.mode == MODE_AG && tm / tiles_per_rank != c.rank) {
          // remote rows: wait until the copy drivers have landed this tile in local memory
          // (multicast: the flag was bumped by the sending rank, so the poll is system scope)
          if (!wait_u32_ge(&p.ready[tm], p.epoch, p.mc != nullptr, status, ST_TIMEOUT_PEER, abort_flag, c.wait_ns)) {
            ok = false;
            break;
          }
          fence_proxy_async_all();
        }
        const int m0 = tm * FG_BM, n0 = tn * BN;
        for (int kb_ = 0; kb_ < nk; ++kb_, ++it) {
          const int s = it % FG_STAGES;
          const uint32_t ph = (it / FG_STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * S::STAGE_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full[s], kb_ * FG_BK, m0);
          if constexpr (!B_MN) {
            tma_load_2d(a_dst + S::A_BYTES, &tmB, &full[s], kb_ * FG_BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(a_dst + S::A_BYTES + j * 8192, &tmB, &full[s], n0 + 64 * j, kb_ * FG_BK);
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_bf16(FG_BM, BN, false, B_MN);
    uint32_t it = 0, tile_i = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += p.n_gemm, ++tile_i) {
      const uint32_t buf = tile_i & 1u, bph = (tile_i >> 1) & 1u;
      if (!mbar_wait(&tempty[buf], bph ^ 1u, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb_ = 0; kb_ < nk; ++kb_, ++it) {
        const int s = it % FG_STAGES;
        const uint32_t ph = (it / FG_STAGES) & 1u;
        if (!mbar_wait(&full[s], ph, abort_flag, status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < FG_BK / 16; ++k)
            umma_ss(d_tmem, make_smem_desc(a_addr + k * 32, 16, 1024),
                    B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024),
                    idesc, (kb_ > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (kb_ == nk - 1) umma_commit(&tfull[buf]);
        }
        __syncwarp();
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tile_i = 0;
    bool ok = true;
    bool go_seen = false;
    // reduce-scatter: counters of remote tiles whose stores are out but not yet published.  One
    // system-scope fence then covers several tiles (a fence waits for the acknowledgements of all
    // earlier peer stores, i.e. an NVLink round trip); owners only read their tiles at the end of
    // their own walk, so publishing a few tiles late costs nothing.
    constexpr int PUB_BATCH = 4;
    uint32_t* pub[PUB_BATCH];
    int n_pub = 0;
    bool tma_busy = false;      // this warp's lane 0 has TMA stores that may still read the staging buffers
    auto publish = [&]() {
      if (lane == 0 && n_pub > 0) {
        tma_store_wait<0>();    // the tiles' TMA stores have been performed
        fence_sys();
        for (int i = 0; i < n_pub; ++i) red_relaxed_sys_add_u32(pub[i], 1u);
      }
      n_pub = 0;
    };
    for (int t = cta; t < num_tiles && ok; t += p.n_gemm, ++tile_i) {
      const uint32_t buf = tile_i & 1u, bph = (tile_i >> 1) & 1u;
      int tm, tn;
      coords(t, tm, tn);
      const int m0 = tm * FG_BM, n0 = tn * BN;
      if (!mbar_wait(&tfull[buf], bph, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
      __nv_bfloat16* cbase;        // row 0 of this warp's 32 rows in the destination
      bool own = false;            // reduce-scatter: tile of this rank's own rows
      bool own_mc = false;         // ... in the multicast variant (summed fetch after the local store)
      if (p.mode == MODE_RS) {
        if (!go_seen) {
          if (!wait_u32_ge(p.go, p.epoch, false, status, ST_TIMEOUT_PEER, abort_flag, c.wait_ns)) { ok = false; break; }
          go_seen = true;
        }
        const int owner = tm / tiles_per_rank;
        own = owner == c.rank;
        if (own) {          // the own rows come last: everything still unpublished goes out first
          __syncwarp();
          publish();
        }
        if (p.mc != nullptr) {
          // multicast: every partial tile goes to LOCAL staging [M, N]; own tiles are fetched summed below
          cbase = reinterpret_cast<__nv_bfloat16*>(p.uc + p.stage_off) + static_cast<long>(m0 + q * 32) * N;
          own_mc = own;
          own = false;
        } else if (!own) {
          __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(c.base[owner] + p.stage_off) +
                                 static_cast<long>(c.rank) * p.rows_per_rank * N;
          cbase = stage + static_cast<long>(m0 + q * 32 - owner * p.rows_per_rank) * N;
        } else {
          // this rank's own rows come last in its tile order; by then the peers' partial tiles have
          // (normally) landed in the staging slots here, so the sum is finished in this epilogue
          cbase = p.out + static_cast<long>(m0 + q * 32 - owner * p.rows_per_rank) * N;
          bool got = true;
          if (lane < c.world && lane != c.rank) {
            const uint32_t* cnt = reinterpret_cast<const uint32_t*>(c.base[c.rank] + p.cnt_off) +
                                  (static_cast<long>(lane) * tiles_per_rank + (tm - owner * tiles_per_rank)) * tiles_n + tn;
            got = wait_u32_ge(cnt, p.epoch * 4u, true, status, ST_TIMEOUT_PEER, abort_flag, c.wait_ns);
          }
          if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        }
      } else {
        cbase = p.out + static_cast<long>(m0 + q * 32) * N;
      }
      // Accumulator → bf16 → this warp's 4 KB of shared memory (32 rows x 128 B, 16-byte units
      // XOR-swizzled by row) → global/peer memory as full 128-byte row segments.  Writing straight
      // from registers would give every lane its own row, i.e. 16-byte scattered writes, which
      // NVLink carries at a fraction of its bandwidth.
      uint8_t* stg0 = smem + S::TILE_BYTES + q * 8192;
      const bool use_tma = p.mode == MODE_RS && p.push_tma && !own && !own_mc && p.mc == nullptr;
      if (!use_tma && tma_busy) {
        // the lanes are about to write staging buffer 0 themselves: earlier TMA stores must have read it
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        tma_busy = false;
      }
#pragma unroll 1
      for (int cp = 0; cp < BN / 64; ++cp) {
        uint8_t* stg = stg0 + (use_tma ? (cp & 1) * 4096 : 0);
        if (use_tma) {
          // buffer (cp & 1) was handed to the TMA unit two blocks ago: at most the newest store may still read
          if (tma_busy) {
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
          if (n0 + cp * 64 >= N) break;
        }
        // own rows of a reduce-scatter: gather the peers' partial sums of this 32x64 block first, eight
        // independent 16-byte loads per lane and peer in flight, so their latency hides behind the
        // accumulator drain below
        float pacc[8][8];
        if (own) {
#pragma unroll
          for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int b2 = 0; b2 < 8; ++b2) pacc[a][b2] = 0.f;
          const int u = lane & 7;
          const int col = n0 + cp * 64 + u * 8;
          const __nv_bfloat16* st0 = reinterpret_cast<const __nv_bfloat16*>(c.base[c.rank] + p.stage_off);
          const long slot_elems = static_cast<long>(p.rows_per_rank) * N;
          const long off0 = static_cast<long>(m0 + q * 32 + (lane >> 3) - c.rank * p.rows_per_rank) * N + col;
          const bool colok = col + 8 <= N;
#pragma unroll 1
          for (int s2 = 0; s2 < c.world; ++s2) {
            if (s2 == c.rank) continue;
            uint4 pv[8];
#pragma unroll
            for (int it4 = 0; it4 < 8; ++it4) {
              const bool rok = colok && (m0 + q * 32 + it4 * 4 + (lane >> 3) < M);
              pv[it4] = rok ? *reinterpret_cast<const uint4*>(st0 + s2 * slot_elems + off0 + static_cast<long>(it4 * 4) * N)
                            : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int it4 = 0; it4 < 8; ++it4) {
              const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&pv[it4]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 t2 = __bfloat1622float2(x[i]);
                pacc[it4][2 * i] += t2.x;
                pacc[it4][2 * i + 1] += t2.y;
              }
            }
          }
        }
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
        if (use_tma) {
          // the block in shared memory has exactly the layout a 128-byte-swizzled TMA box reads
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int owner = tm / tiles_per_rank;
            tma_store_2d(&stage_maps.m[owner], stg, n0 + cp * 64, m0 + q * 32 - owner * p.rows_per_rank);
            tma_store_commit();
          }
          tma_busy = true;
          continue;
        }
        __syncwarp();
        const int u = lane & 7;
        const int col = n0 + cp * 64 + u * 8;
#pragma unroll
        for (int it4 = 0; it4 < 8; ++it4) {
          const int r = it4 * 4 + (lane >> 3);
          uint4 o = *reinterpret_cast<const uint4*>(stg + r * 128 + ((u ^ (r & 7)) << 4));
          if (m0 + q * 32 + r < M && col + 8 <= N) {
            if (own) {
              const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&o);
              float f[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 t2 = __bfloat1622float2(x[i]);
                f[2 * i] = t2.x + pacc[it4][2 * i];
                f[2 * i + 1] = t2.y + pacc[it4][2 * i + 1];
              }
              o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
            }
            *reinterpret_cast<uint4*>(cbase + static_cast<long>(r) * N + col) = o;
          }
        }
        __syncwarp();
      }
      // the accumulator has been drained: hand the TMEM buffer back before the (slow) system-scope
      // fence, so the MMA warp is not held up by the publication of this tile
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
      if (p.mode == MODE_RS && !own && !own_mc) {
        // publish this warp's 32 rows of the tile to the owner: the lanes' stores are ordered before
        // lane 0 by the warp barrier, and lane 0's system-scope release is cumulative over them
        __syncwarp();
        {
          const int owner = tm / tiles_per_rank;
          pub[n_pub++] = reinterpret_cast<uint32_t*>(c.base[owner] + p.cnt_off) +
                         (static_cast<long>(c.rank) * tiles_per_rank + (tm - owner * tiles_per_rank)) * tiles_n + tn;
          if (n_pub == PUB_BATCH) publish();
        }
        __syncwarp();
      }
      if (own_mc) {
        // own rows, multicast variant: this rank's partial is in local staging; once the peers have
        // published theirs, one multimem.ld_reduce per 16 bytes returns the sum over all ranks
        __syncwarp();
        fence_sys();
        bool got = true;
        if (lane < c.world && lane != c.rank) {
          const uint32_t* cnt = reinterpret_cast<const uint32_t*>(c.base[c.rank] + p.cnt_off) +
                                (static_cast<long>(lane) * tiles_per_rank + (tm - c.rank * tiles_per_rank)) * tiles_n + tn;
          got = wait_u32_ge(cnt, p.epoch * 4u, true, status, ST_TIMEOUT_PEER, abort_flag, c.wait_ns);
        }
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        const __nv_bfloat16* mrow = reinterpret_cast<const __nv_bfloat16*>(p.mc + p.stage_off) +
                                    static_cast<long>(m0 + q * 32) * N;
        __nv_bfloat16* orow = p.out + static_cast<long>(m0 + q * 32 - c.rank * p.rows_per_rank) * N;
        const int u = lane & 7;
#pragma unroll 1
        for (int cp = 0; cp < BN / 64; ++cp) {
          const int col = n0 + cp * 64 + u * 8;
          if (col + 8 > N) continue;
          uint4 sv[8];
#pragma unroll
          for (int it4 = 0; it4 < 8; ++it4) {
            const int r = it4 * 4 + (lane >> 3);
            sv[it4] = (m0 + q * 32 + r < M) ? mm_ld_reduce_bf16x8(mrow + static_cast<long>(r) * N + col)
                                            : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int it4 = 0; it4 < 8; ++it4) {
            const int r = it4 * 4 + (lane >> 3);
            if (m0 + q * 32 + r < M) *reinterpret_cast<uint4*>(orow + static_cast<long>(r) * N + col) = sv[it4];
          }
        }
      }
    }
    // tiles published late must still go out when this CTA has no own tile after them (also on the
    // error path: the stores were made, and peers should not wait longer than needed)
    __syncwarp();
    publish();
    if (lane == 0) tma_store_wait<0>();      // nothing of this CTA's shared memory is still being read
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, bool B_MN>
static int launch_fused(const void* A, const void* W, const FusedParams& p, int M, int N, int K, int lda, int ldw,
                        cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, FG_BK, FG_BM);
  if (rc) return rc;
  StageMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (p.mode == MODE_RS && p.push_tma) {
    // this rank's slot in every peer's staging area: [rows_per_rank, N] bf16, blocks of 32 rows x 64 columns
    for (int r = 0; r < p.peer.world; ++r) {
      if (r == p.peer.rank) continue;
      const uint8_t* base = p.peer.base[r] + p.stage_off + static_cast<uint64_t>(p.peer.rank) * p.rows_per_rank * N * 2;
      rc = make_tmap_2d_bf16(&maps.m[r], base, N, p.rows_per_rank, N, 64, 32);
      if (rc) return rc;
    }
  }
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, W, K, N, ldw, FG_BK, BN);
  else       rc = make_tmap_2d_bf16(&tmB, W, N, K, ldw, 64, FG_BK);
  if (rc) return rc;
  auto kern = fused_gemm_kernel<BN, B_MN>;
  constexpr int smem = FgSmem<BN>::TOTAL > (FG_SLOTS * FG_CHUNK + 2048) ? FgSmem<BN>::TOTAL : (FG_SLOTS * FG_CHUNK + 2048);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  const int grid = p.n_first + p.n_gemm + p.n_last;
  KB_LAUNCH_EPOCH(kern, grid, FG_THREADS, smem, stream,
                  (EpochLoc{3, static_cast<int>(offsetof(FusedParams, epoch)), 4}), tmA, tmB, maps, p, M, N, K);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}

static PeerCtx fused_ctx(void* const* bases, int rank, int world, uint64_t flag_off, int* status) {
  PeerCtx c;
  for (int i = 0; i < MAX_PEERS; ++i) c.base[i] = i < world ? reinterpret_cast<uint8_t*>(bases[i]) : nullptr;
  c.rank = rank; c.world = world; c.flag_off = flag_off; c.status = status;
  c.wait_ns = peer_wait_limit_ns();
  return c;
}

}  // namespace kb

using namespace kb;

// Y[M,N] = gathered(X)[M,K] · op(W) with W stored [N,K] (b_mn = 0) or [K,N] (b_mn = 1), where this rank's shard already sits at rows
// [rank*Ms, (rank+1)*Ms) of the gathered buffer at heap offset xg_off (same offset on all ranks).
// ready: local uint32[M/128] flags (persist across calls, epoch-valued).  n_comm copy-driver CTAs.
static int ag_gemm_impl(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t xg_off, const void* W,
                       void* Y, int M, int N, int K, int ldw, int b_mn, uint32_t* ready, uint32_t epoch, int n_comm,
                       int num_sms, int* status, cudaStream_t stream, uint8_t* uc, uint8_t* mc, uint64_t ready_off,
                       void* xg_local = nullptr) {
  if (world < 2 || world > MAX_PEERS || M % (world * FG_BM) || (K & 7) || (xg_off & 1023)) return ST_BAD_ARG;
  if (xg_local && (mc || (reinterpret_cast<uintptr_t>(xg_local) & 15))) return ST_BAD_ARG;
  if (num_sms <= 0) num_sms = device_sm_count();
  if (n_comm < 1) n_comm = 1;
  if (n_comm > MAX_SIGNAL_CTAS) n_comm = MAX_SIGNAL_CTAS;
  if (n_comm > num_sms / 2) n_comm = num_sms / 2;
  FusedParams p{};
  p.peer = fused_ctx(bases, rank, world, flag_off, status);
  p.mode = MODE_AG;
  p.n_first = n_comm;
  p.n_last = 0;
  p.rows_per_rank = M / world;
  p.epoch = epoch;
  p.xg_off = xg_off;
  p.ready = mc ? reinterpret_cast<uint32_t*>(uc + ready_off) : ready;
  p.out = reinterpret_cast<__nv_bfloat16*>(Y);
  p.uc = uc; p.mc = mc; p.ready_off = ready_off;
  p.xg_local = reinterpret_cast<uint8_t*>(xg_local);
  const void* A = xg_local ? xg_local : mc ? uc + xg_off : reinterpret_cast<const uint8_t*>(bases[rank]) + xg_off;
  const bool narrow = (N <= 128) || (N % 256 != 0 && N % 256 <= 128);
  const int bn = narrow ? 128 : 256;
  const int tiles = (M / FG_BM) * ((N + bn - 1) / bn);
  p.n_gemm = num_sms - n_comm < tiles ? num_sms - n_comm : tiles;
  if (narrow) return b_mn ? launch_fused<128, true>(A, W, p, M, N, K, K, ldw, stream)
                          : launch_fused<128, false>(A, W, p, M, N, K, K, ldw, stream);
  return b_mn ? launch_fused<256, true>(A, W, p, M, N, K, K, ldw, stream)
              : launch_fused<256, false>(A, W, p, M, N, K, K, ldw, stream);
}

extern "C" int kb_ag_gemm_bf16(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t xg_off,
                               const void* W, void* Y, int M, int N, int K, int ldw, int b_mn, uint32_t* ready,
                               uint32_t epoch, int n_comm, int num_sms, int* status, cudaStream_t stream) {
  return ag_gemm_impl(bases, rank, world, flag_off, xg_off, W, Y, M, N, K, ldw, b_mn, ready, epoch, n_comm, num_sms,
                      status, stream, nullptr, nullptr, 0);
}

// Same, with the gathered buffer in ordinary local memory (`xg_local`, [M, K], this rank's rows already filled
// in): every rank's own shard sits in a [M/world, K] buffer at heap offset shard_off, the copy drivers pull the
// peers' shards from there into xg_local.  The caller may keep xg_local (the weight-gradient GEMM of the
// backward pass reads it) without copying it out of the heap.
extern "C" int kb_ag_gemm_local_bf16(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t shard_off,
                                     void* xg_local, const void* W, void* Y, int M, int N, int K, int ldw, int b_mn,
                                     uint32_t* ready, uint32_t epoch, int n_comm, int num_sms, int* status,
                                     cudaStream_t stream) {
  if (!xg_local) return ST_BAD_ARG;
  return ag_gemm_impl(bases, rank, world, flag_off, shard_off, W, Y, M, N, K, ldw, b_mn, ready, epoch, n_comm, num_sms,
                      status, stream, nullptr, nullptr, 0, xg_local);
}

// Switch-multicast variant: the gathered buffer (xg_off) and the per-tile ready flags (ready_off, uint32 per
// 128 rows, zero before the channel's first call) live inside an NVLS buffer whose local view is `uc` and whose
// multicast view is `mc`; this rank's shard already sits in its rows of the local gathered buffer.  `epoch`
// must be the number of calls made on this channel (flags count calls).
extern "C" int kb_ag_gemm_mc_bf16(void* const* bases, int rank, int world, uint64_t flag_off, void* uc, void* mc,
                                  uint64_t xg_off, uint64_t ready_off, const void* W, void* Y, int M, int N, int K,
                                  int ldw, int b_mn, uint32_t epoch, int n_comm, int num_sms, int* status,
                                  cudaStream_t stream) {
  if (!uc || !mc || (ready_off & 3)) return ST_BAD_ARG;
  return ag_gemm_impl(bases, rank, world, flag_off, xg_off, W, Y, M, N, K, ldw, b_mn, nullptr, epoch, n_comm, num_sms,
                      status, stream, reinterpret_cast<uint8_t*>(uc), reinterpret_cast<uint8_t*>(mc), ready_off);
}

// out[M/world, N] = rows owned by this rank of sum over ranks of (A[M,K] · op(W)); W as above.
// stage_off: staging [world][M/world][N] bf16; cnt_off: uint32 counters [world][M/world/128][tiles_n];
// go: local uint32 flag.  n_comm: SMs of the num_sms budget that the kernel does not occupy.
static int gemm_rs_impl(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t stage_off,
                       uint64_t cnt_off, const void* A, int lda, const void* W, int ldw, int b_mn, void* out, int M,
                       int N, int K, uint32_t* go, uint32_t epoch, int n_comm, int num_sms, int* status,
                       cudaStream_t stream, uint8_t* uc, uint8_t* mc) {
  if (world < 2 || world > MAX_PEERS || M % (world * FG_BM) || (K & 7) || (N & 7) || (lda & 7)) return ST_BAD_ARG;
  if (num_sms <= 0) num_sms = device_sm_count();
  if (n_comm < 0) n_comm = 0;
  FusedParams p{};
  p.peer = fused_ctx(bases, rank, world, flag_off, status);
  p.mode = MODE_RS;
  p.n_first = 0;
  p.n_last = 1;
  p.rows_per_rank = M / world;
  p.epoch = epoch;
  p.stage_off = stage_off;
  p.cnt_off = cnt_off;
  p.go = go;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.uc = uc; p.mc = mc;
  {
    // TMA push of the partial tiles (KAREUS_RS_TMA=0: the warp's lanes store them); needs 16-byte rows
    static const bool want = [] { const char* e = getenv("KAREUS_RS_TMA"); return !(e && e[0] == '0'); }();
    p.push_tma = (want && mc == nullptr && (N & 7) == 0 && (stage_off & 15) == 0) ? 1 : 0;
  }
  const bool narrow = (N <= 128) || (N % 256 != 0 && N % 256 <= 128);
  const int bn = narrow ? 128 : 256;
  const int tiles = (M / FG_BM) * ((N + bn - 1) / bn);
  // one CTA runs the start barrier; n_comm SMs stay free for the other stream's kernels
  int budget = num_sms - 1 - n_comm;
  if (budget < 8) budget = 8;
  p.n_gemm = budget < tiles ? budget : tiles;
  if (narrow) return b_mn ? launch_fused<128, true>(A, W, p, M, N, K, lda, ldw, stream)
                          : launch_fused<128, false>(A, W, p, M, N, K, lda, ldw, stream);
  return b_mn ? launch_fused<256, true>(A, W, p, M, N, K, lda, ldw, stream)
              : launch_fused<256, false>(A, W, p, M, N, K, lda, ldw, stream);
}

extern "C" int kb_gemm_rs_bf16(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t stage_off,
                               uint64_t cnt_off, const void* A, int lda, const void* W, int ldw, int b_mn, void* out,
                               int M, int N, int K, uint32_t* go, uint32_t epoch, int n_comm, int num_sms, int* status,
                               cudaStream_t stream) {
  return gemm_rs_impl(bases, rank, world, flag_off, stage_off, cnt_off, A, lda, W, ldw, b_mn, out, M, N, K, go, epoch,
                      n_comm, num_sms, status, stream, nullptr, nullptr);
}

// Switch-multicast variant: stage_off names a [M, N] bf16 staging area inside an NVLS buffer (local view
// `uc`, multicast view `mc`); the tile counters (cnt_off) stay in the peer-mapped heap.
extern "C" int kb_gemm_rs_mc_bf16(void* const* bases, int rank, int world, uint64_t flag_off, void* uc, void* mc,
                                  uint64_t stage_off, uint64_t cnt_off, const void* A, int lda, const void* W, int ldw,
                                  int b_mn, void* out, int M, int N, int K, uint32_t* go, uint32_t epoch, int n_comm,
                                  int num_sms, int* status, cudaStream_t stream) {
  if (!uc || !mc || (stage_off & 15)) return ST_BAD_ARG;
  return gemm_rs_impl(bases, rank, world, flag_off, stage_off, cnt_off, A, lda, W, ldw, b_mn, out, M, N, K, go, epoch,
                      n_comm, num_sms, status, stream, reinterpret_cast<uint8_t*>(uc), reinterpret_cast<uint8_t*>(mc));
}

// Number of column tiles the fused kernels use for a given N (sizes the counter array).
extern "C" int kb_fused_tiles_n(int N) {
  const bool narrow = (N <= 128) || (N % 256 != 0 && N % 256 <= 128);
  const int bn = narrow ? 128 : 256;
  return (N + bn - 1) / bn;
}
