// Device-side primitives for kernels that move data between GPUs of one NVSwitch domain through
// peer-mapped memory (plain loads/stores over NVLink; no TMA multicast, no multimem).
//
// Signalling uses monotone 64-bit tokens: a rank publishes `value` with a system-scope release
// store into a slot in the peer's memory; the peer polls its own slot with acquire loads until it
// sees a value >= the one it expects.  Tokens only grow (the host passes a per-channel epoch), so
// slots never need resetting.  Every poll is bounded by wall time: on expiry the waiter writes
// ST_TIMEOUT_PEER to the status word and returns false, and the kernel winds down instead of
// hanging.  (The reference's device semaphores have the same token protocol but trap the GPU with
// a device assert when their spin limit is hit: 3rdparty/mscclpp/include/mscclpp/
// semaphore_device.hpp:61-149, poll_device.hpp:12-18.)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "sm100.cuh"

namespace kb {

constexpr int MAX_PEERS = 8;
constexpr int MAX_SIGNAL_CTAS = 64;   // CTAs of a kernel that take part in peer barriers

struct PeerCtx {
  uint8_t* base[MAX_PEERS];   // heap base of every rank in this rank's address space
  int rank;
  int world;
  uint64_t flag_off;          // byte offset (inside each heap) of this channel's flag block:
                              // uint64 flags[MAX_PEERS][MAX_SIGNAL_CTAS]
  int* status;
  uint64_t wait_ns;           // bound of every wait on another GPU (host: peer_wait_limit_ns())
};

// Bound of a wait for a peer, in ns.  A peer may legitimately be late by as much as the kernels that
// are queued in front of its matching launch need (another nanobatch's GEMM can hold every SM), so the
// limit is a run-time setting: KAREUS_PEER_WAIT_MS (default 2000) or kb_set_peer_wait_ms().
uint64_t peer_wait_limit_ns();

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ----------------------------------------------------------------------------- NVLink-switch multicast
// `mc` addresses are views of a multicast object that every rank of the group has bound memory to
// (parallel/nvls.py).  ld_reduce returns the element-wise sum of all ranks' copies, computed in the
// switch; st writes all copies; red adds to all copies.
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_bf16x8(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void mm_red_add_u32(void* mc, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Bounded polls.  `abort_flag` may be null (kernels without a CTA-wide abort flag).
__device__ __forceinline__ bool wait_u64_ge(const uint64_t* p, uint64_t want, int* status, int code,
                                            volatile int* abort_flag = nullptr, uint64_t limit_ns = KB_WAIT_NS) {
  if (ld_acquire_sys(p) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_sys(p) < want) {
    if ((++spins & 31u) == 0u) {
      if (abort_flag && *abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        if (abort_flag) *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool wait_u32_ge(const uint32_t* p, uint32_t want, bool sys_scope, int* status, int code,
                                            volatile int* abort_flag = nullptr, uint64_t limit_ns = KB_WAIT_NS) {
  auto ld = [&]() { return sys_scope ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p); };
  if (static_cast<int32_t>(ld() - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld() - want) < 0) {
    if ((++spins & 31u) == 0u) {
      if (abort_flag && *abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        if (abort_flag) *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Barrier among the CTAs with index `cta` of all ranks (the same grid must run on every rank).
// Everything this CTA wrote before the call is visible to the peers after it.  Returns false on
// timeout (every thread of the CTA gets the same answer).
__device__ __forceinline__ bool peer_barrier(const PeerCtx& c, int cta, uint64_t value, int* smem_ok) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) *smem_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    uint64_t* remote = reinterpret_cast<uint64_t*>(c.base[peer] + c.flag_off) + c.rank * MAX_SIGNAL_CTAS + cta;
    st_release_sys(remote, value);
    const uint64_t* mine = reinterpret_cast<const uint64_t*>(c.base[c.rank] + c.flag_off) + peer * MAX_SIGNAL_CTAS + cta;
    if (!wait_u64_ge(mine, value, c.status, ST_TIMEOUT_PEER, nullptr, c.wait_ns)) *smem_ok = 0;
  }
  __syncthreads();
  return *smem_ok != 0;
}

}  // namespace kb
