// Kernel launches of this library go through kb::launch(), which can also RECORD them.
//
// A training step enqueues tens of thousands of kernels whose arguments do not change from one
// microbatch to the next (same buffers, same shapes, same weights).  While a recording is open,
// every launch, device-to-device copy, memset, event record and stream wait issued through this
// header is appended to a launch list: the kernel's function pointer, its grid/block/shared-memory
// shape, a private copy of its argument values (tensor maps included) and the stream it ran on.
// kb_replay() then re-issues the whole list from C++ with no interpreter in the loop, on the same
// streams and with the same event edges, so the order in which kernels that wait on peer GPUs are
// started stays exactly what it was when the list was recorded.
//
// Per-call values: kernels of the peer-memory token protocol take a channel epoch that must grow
// by one on every call.  The host keeps that counter in memory it names with
// kb_rec_next_epoch(&counter) just before the call; the launch site says where the epoch sits in
// the kernel's arguments (EpochLoc), and a replay increments the counter and patches the copy of
// the arguments before launching.
//
// This is the role CUDA graphs play elsewhere; an own list keeps explicit control of stream
// assignment (two peer-waiting kernels must be started in the same order on every rank) and lets
// the epochs be patched without per-node update calls.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <tuple>
#include <type_traits>
#include <utility>

namespace kb {

struct EpochLoc {
  int arg;        // index of the kernel argument that holds the epoch, -1: none
  int offset;     // byte offset inside that argument
  int size;       // 4 or 8 bytes
};
constexpr EpochLoc NO_EPOCH{-1, 0, 0};

extern bool g_recording;   // set between kb_rec_begin and kb_rec_end

void record_launch(const void* func, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void* const* args,
                   const size_t* sizes, const size_t* aligns, int nargs, EpochLoc epoch);
void record_memcpy(void* dst, const void* src, size_t bytes, cudaStream_t stream);
void record_memset(void* dst, int value, size_t bytes, cudaStream_t stream);

template <typename... KArgs, typename... Args, size_t... I>
inline cudaError_t launch_impl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               EpochLoc epoch, std::index_sequence<I...>, Args&&... args) {
  std::tuple<std::decay_t<KArgs>...> vals(static_cast<std::decay_t<KArgs>>(std::forward<Args>(args))...);
  void* ptrs[sizeof...(KArgs) > 0 ? sizeof...(KArgs) : 1] = {static_cast<void*>(&std::get<I>(vals))...};
  if (g_recording) {
    static const size_t sizes[] = {sizeof(std::decay_t<KArgs>)..., 0};
    static const size_t aligns[] = {alignof(std::decay_t<KArgs>)..., 0};
    record_launch(reinterpret_cast<const void*>(kernel), grid, block, smem, stream, ptrs, sizes, aligns,
                  static_cast<int>(sizeof...(KArgs)), epoch);
  }
  return cudaLaunchKernel(reinterpret_cast<const void*>(kernel), grid, block, ptrs, smem, stream);
}

// kernel<<<grid, block, smem, stream>>>(args...) that is also recordable.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          EpochLoc epoch, Args&&... args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "argument count differs from the kernel's parameter list");
  return launch_impl(kernel, grid, block, smem, stream, epoch, std::index_sequence_for<KArgs...>{},
                     std::forward<Args>(args)...);
}

// cudaMemcpyAsync (device to device) / cudaMemsetAsync that are also recordable.
inline cudaError_t memcpy_d2d(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  if (g_recording) record_memcpy(dst, src, bytes, stream);
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}
inline cudaError_t memset_async(void* dst, int value, size_t bytes, cudaStream_t stream) {
  if (g_recording) record_memset(dst, value, bytes, stream);
  return cudaMemsetAsync(dst, value, bytes, stream);
}

}  // namespace kb

#define KB_LAUNCH(kernel, grid, block, smem, stream, ...) \
  kb::launch(kernel, dim3(grid), dim3(block), smem, stream, kb::NO_EPOCH, __VA_ARGS__)
#define KB_LAUNCH_EPOCH(kernel, grid, block, smem, stream, epoch_loc, ...) \
  kb::launch(kernel, dim3(grid), dim3(block), smem, stream, epoch_loc, __VA_ARGS__)
