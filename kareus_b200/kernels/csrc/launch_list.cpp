// Launch lists: record a sequence of kernel launches, copies, memsets and stream/event edges
// once, replay it from C++ (see launch.h for why and what is patched per replay).
//
// C ABI (all return 0 or a positive error code unless noted):
//   kb_rec_begin(compute_stream)        open a recording; returns a list id > 0 (or < 0 on error).
//                                       Work recorded on `compute_stream` is replayed on whatever
//                                       stream kb_replay is given; other streams keep their handle.
//   kb_rec_end()                        close it; returns the number of recorded operations.
//   kb_rec_abort()                      close and discard the open recording.
//   kb_rec_new_event()                  an event owned by the open list; returns its index.
//   kb_rec_event_record(ev, stream)     note "record ev on stream"   (the caller performs the real one).
//   kb_rec_stream_wait(stream, ev)      note "stream waits for ev"   (likewise).
//   kb_rec_next_epoch(&counter)         the next recorded launch that declares an epoch location takes
//                                       its epoch from this host counter (incremented on every replay).
//   kb_replay(list, compute_stream)     enqueue the whole list.
//   kb_rec_launches(list)               kernels in the list (for launch accounting).
//   kb_rec_free(list)
#include "launch.h"

#include <stdlib.h>
#include <string.h>
#include <memory>
#include <vector>

namespace kb {

bool g_recording = false;

namespace {

enum OpKind : int { OP_LAUNCH = 0, OP_MEMCPY = 1, OP_MEMSET = 2, OP_EVENT_RECORD = 3, OP_STREAM_WAIT = 4 };

struct Op {
  OpKind kind;
  int stream;                 // index into LaunchList::streams (0 = the replay's compute stream)
  // launch
  const void* func = nullptr;
  dim3 grid, block;
  size_t smem = 0;
  size_t args_off = 0;        // first argument pointer in LaunchList::argptrs
  int nargs = 0;
  // epoch patch
  uint64_t* epoch_counter = nullptr;
  size_t epoch_blob_off = 0;
  int epoch_size = 0;
  // memcpy / memset
  void* dst = nullptr;
  const void* src = nullptr;
  size_t bytes = 0;
  int value = 0;
  // events
  int event = -1;
};

struct LaunchList {
  std::vector<Op> ops;
  std::vector<uint8_t> blob;            // argument values; offsets are fixed up into pointers at the end
  std::vector<size_t> arg_offsets;      // per argument: offset into blob
  std::vector<void*> argptrs;           // per argument: pointer into blob (valid after finish())
  std::vector<cudaStream_t> streams;    // [0] is a placeholder for the compute stream
  std::vector<cudaEvent_t> events;
  long launches = 0;
  bool finished = false;

  int stream_index(cudaStream_t s, cudaStream_t compute) {
    if (s == compute) return 0;
    for (size_t i = 1; i < streams.size(); ++i)
      if (streams[i] == s) return static_cast<int>(i);
    streams.push_back(s);
    return static_cast<int>(streams.size() - 1);
  }
  ~LaunchList() {
    for (cudaEvent_t e : events) cudaEventDestroy(e);
  }
};

std::vector<std::unique_ptr<LaunchList>> g_lists;   // index = id - 1
LaunchList* g_open = nullptr;
cudaStream_t g_compute = nullptr;
uint64_t* g_next_epoch = nullptr;

}  // namespace

void record_launch(const void* func, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void* const* args,
                   const size_t* sizes, const size_t* aligns, int nargs, EpochLoc epoch) {
  LaunchList* L = g_open;
  if (!L) return;
  Op op;
  op.kind = OP_LAUNCH;
  op.stream = L->stream_index(stream, g_compute);
  op.func = func;
  op.grid = grid;
  op.block = block;
  op.smem = smem;
  op.args_off = L->arg_offsets.size();
  op.nargs = nargs;
  for (int i = 0; i < nargs; ++i) {
    const size_t al = aligns[i] < 16 ? 16 : aligns[i];
    size_t off = (L->blob.size() + al - 1) / al * al;
    L->blob.resize(off + sizes[i]);
    memcpy(L->blob.data() + off, args[i], sizes[i]);
    L->arg_offsets.push_back(off);
    if (i == epoch.arg && g_next_epoch != nullptr) {
      op.epoch_counter = g_next_epoch;
      op.epoch_blob_off = off + static_cast<size_t>(epoch.offset);
      op.epoch_size = epoch.size;
    }
  }
  if (epoch.arg >= 0) g_next_epoch = nullptr;
  L->ops.push_back(op);
  ++L->launches;
}

void record_memcpy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  LaunchList* L = g_open;
  if (!L) return;
  Op op;
  op.kind = OP_MEMCPY;
  op.stream = L->stream_index(stream, g_compute);
  op.dst = dst;
  op.src = src;
  op.bytes = bytes;
  L->ops.push_back(op);
}

void record_memset(void* dst, int value, size_t bytes, cudaStream_t stream) {
  LaunchList* L = g_open;
  if (!L) return;
  Op op;
  op.kind = OP_MEMSET;
  op.stream = L->stream_index(stream, g_compute);
  op.dst = dst;
  op.value = value;
  op.bytes = bytes;
  L->ops.push_back(op);
}

}  // namespace kb

using namespace kb;

extern "C" int kb_rec_begin(cudaStream_t compute_stream) {
  if (g_open) return -1;
  g_lists.emplace_back(new LaunchList());
  g_open = g_lists.back().get();
  g_open->streams.push_back(nullptr);
  g_compute = compute_stream;
  g_next_epoch = nullptr;
  g_recording = true;
  return static_cast<int>(g_lists.size());
}

static void close_recording() {
  g_recording = false;
  g_open = nullptr;
  g_next_epoch = nullptr;
}

extern "C" long kb_rec_end() {
  LaunchList* L = g_open;
  if (!L) return -1;
  // the blob no longer grows: turn argument offsets into pointers.  Overaligned arguments (tensor
  // maps want 64 bytes) need an aligned base, so move the blob into an aligned allocation.
  const size_t n = L->blob.size();
  std::vector<uint8_t> grown(n + 128);
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(grown.data()) + 127) & ~uintptr_t(127));
  memcpy(base, L->blob.data(), n);
  const size_t shift = static_cast<size_t>(base - grown.data());
  L->blob.swap(grown);
  L->argptrs.resize(L->arg_offsets.size());
  for (size_t i = 0; i < L->arg_offsets.size(); ++i) L->argptrs[i] = L->blob.data() + shift + L->arg_offsets[i];
  for (Op& op : L->ops)
    if (op.epoch_counter) op.epoch_blob_off += shift;
  L->finished = true;
  const long count = static_cast<long>(L->ops.size());
  close_recording();
  return count;
}

extern "C" int kb_rec_abort() {
  if (!g_open) return 0;
  close_recording();
  g_lists.back().reset();
  return 0;
}

extern "C" int kb_rec_new_event() {
  LaunchList* L = g_open;
  if (!L) return -1;
  cudaEvent_t e;
  if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return -2;
  L->events.push_back(e);
  return static_cast<int>(L->events.size() - 1);
}

extern "C" int kb_rec_event_record(int ev, cudaStream_t stream) {
  LaunchList* L = g_open;
  if (!L || ev < 0 || ev >= static_cast<int>(L->events.size())) return 7;
  Op op;
  op.kind = OP_EVENT_RECORD;
  op.stream = L->stream_index(stream, g_compute);
  op.event = ev;
  L->ops.push_back(op);
  return 0;
}

extern "C" int kb_rec_stream_wait(cudaStream_t stream, int ev) {
  LaunchList* L = g_open;
  if (!L || ev < 0 || ev >= static_cast<int>(L->events.size())) return 7;
  Op op;
  op.kind = OP_STREAM_WAIT;
  op.stream = L->stream_index(stream, g_compute);
  op.event = ev;
  L->ops.push_back(op);
  return 0;
}

extern "C" int kb_rec_next_epoch(uint64_t* counter) {
  g_next_epoch = g_recording ? counter : nullptr;
  return 0;
}

extern "C" int kb_rec_active() { return g_recording ? 1 : 0; }

extern "C" int kb_replay(int list, cudaStream_t compute_stream) {
  if (list < 1 || list > static_cast<int>(g_lists.size())) return 7;
  LaunchList* L = g_lists[list - 1].get();
  if (!L || !L->finished || g_recording) return 7;
  L->streams[0] = compute_stream;
  cudaError_t e = cudaSuccess;
  for (const Op& op : L->ops) {
    cudaStream_t st = L->streams[op.stream];
    switch (op.kind) {
      case OP_LAUNCH: {
        if (op.epoch_counter) {
          const uint64_t v = ++(*op.epoch_counter);
          uint8_t* at = L->blob.data() + op.epoch_blob_off;
          if (op.epoch_size == 8) {
            memcpy(at, &v, 8);
          } else {
            const uint32_t v32 = static_cast<uint32_t>(v);
            memcpy(at, &v32, 4);
          }
        }
        e = cudaLaunchKernel(op.func, op.grid, op.block, L->argptrs.data() + op.args_off, op.smem, st);
        break;
      }
      case OP_MEMCPY:
        e = cudaMemcpyAsync(op.dst, op.src, op.bytes, cudaMemcpyDeviceToDevice, st);
        break;
      case OP_MEMSET:
        e = cudaMemsetAsync(op.dst, op.value, op.bytes, st);
        break;
      case OP_EVENT_RECORD:
        e = cudaEventRecord(L->events[op.event], st);
        break;
      case OP_STREAM_WAIT:
        e = cudaStreamWaitEvent(st, L->events[op.event], 0);
        break;
    }
    if (e != cudaSuccess) return 2000 + static_cast<int>(e);
  }
  return 0;
}

extern "C" long kb_rec_launches(int list) {
  if (list < 1 || list > static_cast<int>(g_lists.size()) || !g_lists[list - 1]) return -1;
  return g_lists[list - 1]->launches;
}

extern "C" long kb_rec_ops(int list) {
  if (list < 1 || list > static_cast<int>(g_lists.size()) || !g_lists[list - 1]) return -1;
  return static_cast<long>(g_lists[list - 1]->ops.size());
}

extern "C" int kb_rec_free(int list) {
  if (list < 1 || list > static_cast<int>(g_lists.size())) return 7;
  g_lists[list - 1].reset();
  return 0;
}

// Recordable device-to-device copy and memset for callers outside this library's kernels.
extern "C" int kb_memcpy_d2d(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  cudaError_t e = kb::memcpy_d2d(dst, src, bytes, stream);
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}
extern "C" int kb_memset(void* dst, int value, size_t bytes, cudaStream_t stream) {
  cudaError_t e = kb::memset_async(dst, value, bytes, stream);
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}
