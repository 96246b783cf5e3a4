// All-pairs collectives over the symmetric heap: all-reduce, all-gather, reduce-scatter (bf16).
//
// NVSwitch gives every GPU full bandwidth to every peer, so each collective is one-shot all-pairs:
// every rank reads (or writes) each peer directly.  The grid size is the knob a plan entry
// carries ("SMs given to the collective"): `grid = sm_num`, `block = block_size`, one CTA per SM.
// These are the counterparts of the reference's allreduce1 / allgather4 / reducescatter4
// (3rdparty/mscclpp/python/mscclpp_benchmark/allreduce.cu:155-246,481-525,443-478), with bounded
// waits and tails handled (the reference ignores remainder elements).
//
// Also here: the host side of the heap (allocation, CUDA IPC handle exchange is done by the caller).
#include <cuda_bf16.h>
#include "launch.h"
#include <stdlib.h>
#include <string.h>
#include "peer.cuh"

namespace kb {

__device__ __forceinline__ uint4 add_bf16x8(uint4 a, uint4 b) {
  __nv_bfloat162* x = reinterpret_cast<__nv_bfloat162*>(&a);
  const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = __hadd2(x[i], y[i]);
  return a;
}
__device__ __forceinline__ void acc_bf16x8(float (&f)[8], uint4 a) {
  const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(x[i]);
    f[2 * i] += t.x;
    f[2 * i + 1] += t.y;
  }
}
__device__ __forceinline__ uint4 pack_f8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// In-place sum of `n` bf16 elements living at byte offset `off` of every rank's heap.
// Rank r reduces slice r (fp32 accumulation) and writes the result to every rank.
__global__ void __launch_bounds__(1024, 1)
allreduce_kernel(PeerCtx c, uint64_t off, long n, uint64_t epoch) {
  __shared__ int ok;
  if (!peer_barrier(c, blockIdx.x, epoch * 4 + 1, &ok)) return;
  const long nvec = n >> 3;                      // 16-byte vectors
  const long per = (nvec + c.world - 1) / c.world;
  const long lo = per * c.rank, hi = min(nvec, lo + per);
  for (long i = lo + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 1
    for (int p = 0; p < c.world; ++p) {
      const int src = (c.rank + p) % c.world;
      acc_bf16x8(f, reinterpret_cast<const uint4*>(c.base[src] + off)[i]);
    }
    const uint4 r = pack_f8(f);
#pragma unroll 1
    for (int p = 0; p < c.world; ++p) {
      const int dst = (c.rank + p) % c.world;
      reinterpret_cast<uint4*>(c.base[dst] + off)[i] = r;
    }
  }
  // tail elements (n not a multiple of 8): rank 0 handles them
  if (c.rank == 0 && blockIdx.x == 0) {
    for (long i = (nvec << 3) + threadIdx.x; i < n; i += blockDim.x) {
      float s = 0.f;
      for (int p = 0; p < c.world; ++p) s += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(c.base[p] + off)[i]);
      for (int p = 0; p < c.world; ++p) reinterpret_cast<__nv_bfloat16*>(c.base[p] + off)[i] = __float2bfloat16(s);
    }
  }
  peer_barrier(c, blockIdx.x, epoch * 4 + 2, &ok);
}

// Every rank's shard (`shard_bytes` at offset off + rank*shard_bytes of its own heap) is pulled
// into the same position of this rank's heap.
__global__ void __launch_bounds__(1024, 1)
allgather_kernel(PeerCtx c, uint64_t off, long shard_bytes, uint64_t epoch) {
  __shared__ int ok;
  if (!peer_barrier(c, blockIdx.x, epoch * 4 + 1, &ok)) return;
  const long nvec = shard_bytes >> 4;
  for (int p = 1; p < c.world; ++p) {
    const int src = (c.rank + p) % c.world;
    const uint4* from = reinterpret_cast<const uint4*>(c.base[src] + off + src * shard_bytes);
    uint4* to = reinterpret_cast<uint4*>(c.base[c.rank] + off + src * shard_bytes);
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<long>(gridDim.x) * blockDim.x)
      to[i] = from[i];
  }
  peer_barrier(c, blockIdx.x, epoch * 4 + 2, &ok);
}

// Input: `world` shards of `shard_elems` bf16 at offset `off` of every heap.  Output: the sum over
// ranks of shard `rank`, written to `out` (local memory).
__global__ void __launch_bounds__(1024, 1)
reducescatter_kernel(PeerCtx c, uint64_t off, long shard_elems, __nv_bfloat16* __restrict__ out, uint64_t epoch) {
  __shared__ int ok;
  if (!peer_barrier(c, blockIdx.x, epoch * 4 + 1, &ok)) return;
  const long nvec = shard_elems >> 3;
  const uint64_t my = off + static_cast<uint64_t>(c.rank) * shard_elems * 2;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 1
    for (int p = 0; p < c.world; ++p) {
      const int src = (c.rank + p) % c.world;
      acc_bf16x8(f, reinterpret_cast<const uint4*>(c.base[src] + my)[i]);
    }
    reinterpret_cast<uint4*>(out)[i] = pack_f8(f);
  }
  if (blockIdx.x == 0) {
    for (long i = (nvec << 3) + threadIdx.x; i < shard_elems; i += blockDim.x) {
      float s = 0.f;
      for (int p = 0; p < c.world; ++p) s += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(c.base[p] + my)[i]);
      out[i] = __float2bfloat16(s);
    }
  }
  peer_barrier(c, blockIdx.x, epoch * 4 + 2, &ok);
}

// Stream-ordered barrier among ranks: one CTA signals every peer and waits for all of them.
__global__ void barrier_kernel(PeerCtx c, uint64_t epoch) {
  __shared__ int ok;
  peer_barrier(c, 0, epoch * 4 + 3, &ok);
}

// A wait that nothing satisfies: used by the tests of the bounded-wait path.  `slot` is a flag
// nobody writes; the kernel polls it for at most `limit_ns`, records ST_TIMEOUT_PEER and returns.
__global__ void wait_flag_kernel(const uint64_t* slot, uint64_t want, uint64_t limit_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(slot) < want) {
    if (globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0, ST_TIMEOUT_PEER);
      return;
    }
  }
}

static PeerCtx make_ctx(void* const* bases, int rank, int world, uint64_t flag_off, int* status) {
  PeerCtx c;
  for (int i = 0; i < MAX_PEERS; ++i) c.base[i] = i < world ? reinterpret_cast<uint8_t*>(bases[i]) : nullptr;
  c.rank = rank;
  c.world = world;
  c.flag_off = flag_off;
  c.status = status;
  c.wait_ns = peer_wait_limit_ns();
  return c;
}

}  // namespace kb

namespace kb {
static uint64_t g_peer_wait_ns = 0;
uint64_t peer_wait_limit_ns() {
  if (g_peer_wait_ns == 0) {
    const char* e = getenv("KAREUS_PEER_WAIT_MS");
    long ms = e ? atol(e) : 0;
    if (ms <= 0) ms = 2000;
    g_peer_wait_ns = static_cast<uint64_t>(ms) * 1000000ull;
  }
  return g_peer_wait_ns;
}
}  // namespace kb

using namespace kb;

// Bound (ms) of every later wait for another GPU; see peer.cuh.
extern "C" int kb_set_peer_wait_ms(long ms) {
  if (ms <= 0) return 7;
  kb::g_peer_wait_ns = static_cast<uint64_t>(ms) * 1000000ull;
  return 0;
}

static int clamp_grid(int sm_num) { return sm_num < 1 ? 1 : (sm_num > MAX_SIGNAL_CTAS ? MAX_SIGNAL_CTAS : sm_num); }
static int clamp_block(int b) { return b < 32 ? 32 : (b > 1024 ? 1024 : (b / 32) * 32); }
#define KB_RET_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 2000 + (int)e_; } while (0)

extern "C" int kb_allreduce(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t off, long n,
                            uint64_t epoch, int sm_num, int block, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || (off & 15)) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(allreduce_kernel, clamp_grid(sm_num), clamp_block(block), 0, st, (EpochLoc{3, 0, 8}),
                  make_ctx(bases, rank, world, flag_off, status),
                                                                      off, n, epoch);
  KB_RET_LAUNCH();
}
extern "C" int kb_allgather(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t off, long shard_bytes,
                            uint64_t epoch, int sm_num, int block, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || (off & 15) || (shard_bytes & 15)) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(allgather_kernel, clamp_grid(sm_num), clamp_block(block), 0, st, (EpochLoc{3, 0, 8}),
                  make_ctx(bases, rank, world, flag_off, status),
                                                                      off, shard_bytes, epoch);
  KB_RET_LAUNCH();
}
extern "C" int kb_reducescatter(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t off,
                                long shard_elems, void* out, uint64_t epoch, int sm_num, int block, int* status,
                                cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || (off & 15) || ((shard_elems * 2) & 15)) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(reducescatter_kernel, clamp_grid(sm_num), clamp_block(block), 0, st, (EpochLoc{4, 0, 8}),
      make_ctx(bases, rank, world, flag_off, status), off, shard_elems, reinterpret_cast<__nv_bfloat16*>(out), epoch);
  KB_RET_LAUNCH();
}
extern "C" int kb_peer_barrier(void* const* bases, int rank, int world, uint64_t flag_off, uint64_t epoch, int* status,
                               cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(barrier_kernel, 1, 32, 0, st, (EpochLoc{1, 0, 8}), make_ctx(bases, rank, world, flag_off, status), epoch);
  KB_RET_LAUNCH();
}
extern "C" int kb_wait_flag(const void* slot, uint64_t want, uint64_t limit_ns, int* status, cudaStream_t st) {
  KB_LAUNCH(wait_flag_kernel, 1, 1, 0, st, reinterpret_cast<const uint64_t*>(slot), want, limit_ns, status);
  KB_RET_LAUNCH();
}

// ----------------------------------------------------------------------------- heap (host side)
extern "C" int kb_heap_alloc(size_t bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return 1000 + (int)e;
  e = cudaMemset(*out, 0, bytes);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
extern "C" int kb_heap_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : 1; }
extern "C" int kb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return 1000 + (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int kb_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
extern "C" int kb_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : 1; }
