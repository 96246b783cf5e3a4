// NVLink-switch (NVLS) collectives: a multicast object over every rank's buffer and kernels that
// reduce or broadcast THROUGH the switch with multimem instructions.
//
// Host side (driver API, reached through cudaGetDriverEntryPoint so the library does not link
// libcuda): rank 0 creates the multicast object and exports it as a file descriptor, the other ranks
// import it (the descriptor travels over a Unix socket, see parallel/nvls.py), every rank adds its
// device, allocates physical memory, binds it to the object and maps two views:
//   uc   this rank's own memory (ordinary loads/stores, where the producer writes its data),
//   mc   the multicast view: `multimem.ld_reduce` on it returns the SUM of all ranks' copies, computed
//        in the switch; `multimem.st` writes all copies at once.
// Role of the reference's NVLS channel (3rdparty/mscclpp/src/nvls.cc:59-214,
// include/mscclpp/switch_channel_device.hpp:24-157) and of its allreduce6 kernel
// (python/mscclpp_benchmark/allreduce.cu:858-942).
//
// Device side: all-reduce = every rank reduces its slice with ld_reduce and broadcasts the sums with
// multimem.st (each byte crosses a GPU's links once in each direction instead of (world-1)/world·2
// times for reduce-scatter + all-gather over peer loads); reduce-scatter = ld_reduce of the own
// slice into local memory.  Start/end barriers run over the peer-mapped flag block of the symmetric
// heap, with the usual bounded waits.
//
// A process must unbind and unmap before it exits while peers still use the object; parallel/nvls.py
// does that in close() and the multicast path is off unless KAREUS_NVLS=1.
#include "sm100.cuh"
#include "launch.h"
#include "peer.cuh"
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

namespace kb {

// ----------------------------------------------------------------------------- driver entry points
template <typename Fn>
static Fn drv(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}
#define KB_DRV(name) static auto fn_##name = drv<decltype(&name)>(#name); if (!fn_##name) return 3001
#define KB_CU(call) do { CUresult r_ = (call); if (r_ != CUDA_SUCCESS) return 3100 + static_cast<int>(r_); } while (0)

struct NvlsState {
  int dev = 0, world = 0;
  size_t size = 0;                       // bytes bound per device (multiple of the granularity)
  CUmemGenericAllocationHandle mc = 0, mem = 0;
  CUdeviceptr uc_va = 0, mc_va = 0;
  bool added = false, bound = false, uc_mapped = false, mc_mapped = false;
};

static CUmulticastObjectProp mc_prop(int world, size_t size) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = static_cast<unsigned int>(world);
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// ----------------------------------------------------------------------------- kernels
// In-place sum of `n_vec` 16-byte vectors at byte offset `off` of every rank's bound buffer.
__global__ void __launch_bounds__(1024, 1)
nvls_allreduce_kernel(PeerCtx c, uint8_t* mc, uint64_t off, long n_vec, uint64_t epoch) {
  __shared__ int ok;
  if (!peer_barrier(c, blockIdx.x, epoch * 4 + 1, &ok)) return;       // every rank's data is in place
  const long per = (n_vec + c.world - 1) / c.world;
  const long lo = per * c.rank, hi = min(n_vec, lo + per);
  uint4* base = reinterpret_cast<uint4*>(mc + off);
  for (long i = lo + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const uint4 s = mm_ld_reduce_bf16x8(base + i);
    mm_st_bf16x8(base + i, s);
  }
  peer_barrier(c, blockIdx.x, epoch * 4 + 2, &ok);                    // all sums have landed everywhere
}

// out[shard_vec] = sum over ranks of shard `rank` (16-byte vectors) of the bound buffers at `off`.
__global__ void __launch_bounds__(1024, 1)
nvls_reducescatter_kernel(PeerCtx c, const uint8_t* mc, uint64_t off, long shard_vec, uint4* __restrict__ out,
                          uint64_t epoch) {
  __shared__ int ok;
  if (!peer_barrier(c, blockIdx.x, epoch * 4 + 1, &ok)) return;
  const uint4* base = reinterpret_cast<const uint4*>(mc + off) + shard_vec * c.rank;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < shard_vec;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    out[i] = mm_ld_reduce_bf16x8(base + i);
  peer_barrier(c, blockIdx.x, epoch * 4 + 2, &ok);                    // peers may overwrite their buffers now
}

static PeerCtx nvls_ctx(void* const* bases, int rank, int world, uint64_t flag_off, int* status) {
  PeerCtx c;
  for (int i = 0; i < MAX_PEERS; ++i) c.base[i] = i < world ? reinterpret_cast<uint8_t*>(bases[i]) : nullptr;
  c.rank = rank; c.world = world; c.flag_off = flag_off; c.status = status;
  c.wait_ns = peer_wait_limit_ns();
  return c;
}

}  // namespace kb

using namespace kb;

// 1 if the device can take part in switch multicast, 0 if not, > 1 on error.
extern "C" int kb_nvls_supported(int dev) {
  KB_DRV(cuDeviceGet);
  KB_DRV(cuDeviceGetAttribute);
  CUdevice d;
  KB_CU(fn_cuDeviceGet(&d, dev));
  int v = 0;
  KB_CU(fn_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d));
  return v ? 1 : 0;
}

// Rank 0: create the multicast object for `world` devices and at least `bytes` per device; returns its
// state, the rounded size and a file descriptor for the other ranks.
extern "C" int kb_nvls_create(int dev, int world, size_t bytes, void** state_out, size_t* size_out, int* fd_out) {
  KB_DRV(cuMulticastGetGranularity);
  KB_DRV(cuMulticastCreate);
  KB_DRV(cuMemExportToShareableHandle);
  CUmulticastObjectProp p = mc_prop(world, bytes);
  size_t gran = 0;
  KB_CU(fn_cuMulticastGetGranularity(&gran, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  if (gran == 0) return 3002;
  p.size = (bytes + gran - 1) / gran * gran;
  NvlsState* s = new NvlsState();
  s->dev = dev; s->world = world; s->size = p.size;
  CUresult r = fn_cuMulticastCreate(&s->mc, &p);
  if (r != CUDA_SUCCESS) { delete s; return 3100 + static_cast<int>(r); }
  int fd = -1;
  r = fn_cuMemExportToShareableHandle(&fd, s->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { delete s; return 3100 + static_cast<int>(r); }
  *state_out = s; *size_out = s->size; *fd_out = fd;
  return 0;
}

// Other ranks: import the object from the descriptor received from rank 0 (`size` as returned there).
extern "C" int kb_nvls_import(int dev, int world, size_t size, int fd, void** state_out) {
  KB_DRV(cuMemImportFromShareableHandle);
  NvlsState* s = new NvlsState();
  s->dev = dev; s->world = world; s->size = size;
  CUresult r = fn_cuMemImportFromShareableHandle(&s->mc, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) { delete s; return 3100 + static_cast<int>(r); }
  *state_out = s;
  return 0;
}

// Every rank, once: join the multicast team.  All ranks must have done this before any of them binds.
extern "C" int kb_nvls_add_device(void* state) {
  KB_DRV(cuDeviceGet);
  KB_DRV(cuMulticastAddDevice);
  NvlsState* s = static_cast<NvlsState*>(state);
  CUdevice d;
  KB_CU(fn_cuDeviceGet(&d, s->dev));
  KB_CU(fn_cuMulticastAddDevice(s->mc, d));
  s->added = true;
  return 0;
}

// Every rank: allocate this device's memory, bind it and map both views.
extern "C" int kb_nvls_bind(void* state, void** uc_out, void** mc_out) {
  KB_DRV(cuMemCreate);
  KB_DRV(cuMulticastBindMem);
  KB_DRV(cuMemAddressReserve);
  KB_DRV(cuMemMap);
  KB_DRV(cuMemSetAccess);
  NvlsState* s = static_cast<NvlsState*>(state);
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = s->dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  KB_CU(fn_cuMemCreate(&s->mem, s->size, &prop, 0));
  KB_CU(fn_cuMulticastBindMem(s->mc, 0, s->mem, 0, s->size, 0));
  s->bound = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = s->dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  KB_CU(fn_cuMemAddressReserve(&s->uc_va, s->size, 0, 0, 0));
  KB_CU(fn_cuMemMap(s->uc_va, s->size, 0, s->mem, 0));
  s->uc_mapped = true;
  KB_CU(fn_cuMemSetAccess(s->uc_va, s->size, &acc, 1));
  KB_CU(fn_cuMemAddressReserve(&s->mc_va, s->size, 0, 0, 0));
  KB_CU(fn_cuMemMap(s->mc_va, s->size, 0, s->mc, 0));
  s->mc_mapped = true;
  KB_CU(fn_cuMemSetAccess(s->mc_va, s->size, &acc, 1));
  cudaError_t e = cudaMemset(reinterpret_cast<void*>(s->uc_va), 0, s->size);
  if (e != cudaSuccess) return 1000 + static_cast<int>(e);
  *uc_out = reinterpret_cast<void*>(s->uc_va);
  *mc_out = reinterpret_cast<void*>(s->mc_va);
  return 0;
}

// Unmap, unbind and release everything this rank holds (call while the peers are still alive and idle).
extern "C" int kb_nvls_destroy(void* state) {
  KB_DRV(cuDeviceGet);
  KB_DRV(cuMemUnmap);
  KB_DRV(cuMemAddressFree);
  KB_DRV(cuMulticastUnbind);
  KB_DRV(cuMemRelease);
  NvlsState* s = static_cast<NvlsState*>(state);
  if (!s) return 0;
  cudaDeviceSynchronize();
  int rc = 0;
  auto note = [&](CUresult r) { if (r != CUDA_SUCCESS && rc == 0) rc = 3100 + static_cast<int>(r); };
  if (s->mc_mapped) note(fn_cuMemUnmap(s->mc_va, s->size));
  if (s->mc_va) note(fn_cuMemAddressFree(s->mc_va, s->size));
  if (s->uc_mapped) note(fn_cuMemUnmap(s->uc_va, s->size));
  if (s->uc_va) note(fn_cuMemAddressFree(s->uc_va, s->size));
  if (s->bound) {
    CUdevice d;
    note(fn_cuDeviceGet(&d, s->dev));
    note(fn_cuMulticastUnbind(s->mc, d, 0, s->size));
  }
  if (s->mem) note(fn_cuMemRelease(s->mem));
  if (s->mc) note(fn_cuMemRelease(s->mc));
  delete s;
  return rc;
}

static int clamp_g(int sm_num) { return sm_num < 1 ? 1 : (sm_num > MAX_SIGNAL_CTAS ? MAX_SIGNAL_CTAS : sm_num); }
static int clamp_b(int b) { return b < 32 ? 32 : (b > 1024 ? 1024 : (b / 32) * 32); }

// In-place bf16 all-reduce of n elements (multiple of 8) at byte offset `off` of the bound buffers.
// `bases`/`flag_off`: peer-mapped flag block of the symmetric heap that carries the barriers.
extern "C" int kb_nvls_allreduce(void* const* bases, int rank, int world, uint64_t flag_off, void* mc, uint64_t off,
                                 long n, uint64_t epoch, int sm_num, int block, int* status, cudaStream_t st) {
  if (world < 2 || world > MAX_PEERS || (off & 15) || (n & 7) || mc == nullptr) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(nvls_allreduce_kernel, clamp_g(sm_num), clamp_b(block), 0, st, (EpochLoc{4, 0, 8}),
                  nvls_ctx(bases, rank, world, flag_off, status), reinterpret_cast<uint8_t*>(mc), off, n / 8, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

// out[shard_elems] (local, bf16) = sum over ranks of shard `rank` of the bound buffers at `off`.
extern "C" int kb_nvls_reducescatter(void* const* bases, int rank, int world, uint64_t flag_off, const void* mc,
                                     uint64_t off, long shard_elems, void* out, uint64_t epoch, int sm_num, int block,
                                     int* status, cudaStream_t st) {
  if (world < 2 || world > MAX_PEERS || (off & 15) || (shard_elems & 7) || mc == nullptr) return ST_BAD_ARG;
  KB_LAUNCH_EPOCH(nvls_reducescatter_kernel, clamp_g(sm_num), clamp_b(block), 0, st, (EpochLoc{5, 0, 8}),
                  nvls_ctx(bases, rank, world, flag_off, status), reinterpret_cast<const uint8_t*>(mc), off,
                  shard_elems / 8, reinterpret_cast<uint4*>(out), epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}
