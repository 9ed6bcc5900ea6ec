// Context, memory, copies and the name-keyed kernel table of the C ABI
// (include/tessera_b200.h).  The behaviour mirrors what the reference's
// backends give the core (include/tessera/backend.hpp:847-1037; the ROCm
// backend, src/backends/rocm/rocm_backend.cpp, is the model for ordering and
// blocking semantics): one stream per context, stream-ordered launches and
// device-to-device copies, host-to-device copies that return once the host
// bytes are reusable, blocking device-to-host copies.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <string>

#include "context.h"
#include "launch.h"
#include "tessera_b200.h"

namespace {

using tsr::kStageWindow;
using tsr::kStageWindows;

// Floats of split-K scratch and arrival counters every context holds for the
// launches that split k among CTAs and add the chunks themselves.
constexpr size_t kScratchFloats = 4u << 20;  // 16 MiB
constexpr size_t kScratchTickets = 16384;

int map_cuda(cudaError_t e) {
  if (e == cudaSuccess) return tsr::kOk;
  if (e == cudaErrorMemoryAllocation) return tsr::kOutOfMemory;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidDevice) return tsr::kInvalidArgument;
  return tsr::kDeviceError;
}

// One word of pinned, mapped host memory for the whole process: a device wait
// that gives up raises it (pipeline.cuh), tsr_synchronize reads it.
unsigned int* host_error_word() {
  static unsigned int* word = [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
      cudaGetLastError();
      return static_cast<unsigned int*>(nullptr);
    }
    std::memset(p, 0, 64);
    return static_cast<unsigned int*>(p);
  }();
  return word;
}

// Points the kernels of every file at the error word, once per device.
void publish_error_word(int device) {
  static std::mutex mutex;
  static bool done[64] = {};
  std::lock_guard<std::mutex> lock(mutex);
  if (device < 0 || device >= 64 || done[device]) return;
  unsigned int* word = host_error_word();
  if (word == nullptr) return;
  tsr::staged_set_error_word(word);
  tsr::staged_q6k_set_error_word(word);
  tsr::staged_f16_set_error_word(word);
  tsr::umma_set_error_word(word);
  tsr::umma_f8_set_error_word(word);
  done[device] = true;
}

}  // namespace

int tsr_context::fail(cudaError_t e, const char* what) {
  char buf[256];
  std::snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  error = buf;
  return map_cuda(e);
}

int tsr_context::select() {
  // The current device is per host thread and the reference drives one
  // backend from different threads over time (a fresh thread per
  // tensor-parallel step): re-select on every entry.
  // cudaSetDevice on the already-current device is a cheap no-op; no cache
  // is kept because other entry points of the library also switch devices.
  const cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(e, "cudaSetDevice");
  return tsr::kOk;
}

unsigned char* tsr_context::window(int* index) {
  const int i = stage_next;
  stage_next = (stage_next + 1) % kStageWindows;
  if (stage_busy[i]) {
    cudaEventSynchronize(stage_done[i]);
    stage_busy[i] = false;
  }
  *index = i;
  return stage + static_cast<size_t>(i) * kStageWindow;
}

namespace tsr {

// Output ranges written by the last launch of this library, per stream.
bool pdl_allowed_ranges(cudaStream_t stream, const void* const* reads, const size_t* read_bytes, int nreads,
                        const void* const* writes, const size_t* write_bytes, int nwrites) {
  static const bool enabled = [] {
    const char* v = std::getenv("TSR_PDL");
    return v == nullptr || std::atoi(v) != 0;
  }();
  constexpr int kRanges = 12;
  struct Last {
    cudaStream_t stream;
    bool used;
    int count;
    const unsigned char* ptr[kRanges];
    size_t bytes[kRanges];
  };
  static std::mutex mutex;
  static Last table[16] = {};
  std::lock_guard<std::mutex> lock(mutex);
  Last* slot = nullptr;
  for (Last& l : table)
    if (l.used && l.stream == stream) slot = &l;
  bool ok = enabled;
  if (slot != nullptr) {
    for (int i = 0; i < nreads; ++i) {
      const auto* r = static_cast<const unsigned char*>(reads[i]);
      for (int j = 0; j < slot->count; ++j)
        if (r < slot->ptr[j] + slot->bytes[j] && slot->ptr[j] < r + read_bytes[i]) ok = false;  // previous output is our weight
    }
    if (slot->count < 0) ok = false;  // more outputs than the table holds: anything may have been written
  }
  if (slot == nullptr) {
    static int next = 0;
    slot = &table[next];
    next = (next + 1) % 16;
  }
  slot->stream = stream;
  slot->used = true;
  slot->count = nwrites <= kRanges ? nwrites : -1;
  for (int j = 0; j < slot->count; ++j) {
    slot->ptr[j] = static_cast<const unsigned char*>(writes[j]);
    slot->bytes[j] = write_bytes[j];
  }
  return ok;
}

bool pdl_allowed(cudaStream_t stream, const void* read_ptr, size_t read_bytes, const void* out_ptr,
                 size_t out_bytes) {
  return pdl_allowed_ranges(stream, &read_ptr, &read_bytes, 1, &out_ptr, &out_bytes, 1);
}

int allow_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mutex;
  static std::unordered_map<const void*, unsigned long long> done;  // kernel -> device bit mask
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return kDeviceError;
  const unsigned long long bit = 1ull << (dev & 63);
  std::lock_guard<std::mutex> lock(mutex);
  unsigned long long& mask = done[kernel];
  if (mask & bit) return kOk;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return kDeviceError;
  }
  mask |= bit;
  return kOk;
}

}  // namespace tsr

extern "C" {

int tsr_device_count(int* count) {
  if (!count) return tsr::kInvalidArgument;
  *count = 0;
  const cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    return tsr::kDeviceError;
  }
  return tsr::kOk;
}

int tsr_device_name(int device, char* out, size_t capacity) {
  if (!out || capacity == 0) return tsr::kInvalidArgument;
  cudaDeviceProp prop;
  const cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return map_cuda(e);
  }
  std::snprintf(out, capacity, "%s", prop.name);
  return tsr::kOk;
}

static int create_common(int device_index, cudaStream_t borrowed, bool borrow, tsr_context** out) {
  if (!out) return tsr::kInvalidArgument;
  *out = nullptr;
  int count = 0;
  if (tsr_device_count(&count) != tsr::kOk || count == 0) return tsr::kDeviceError;
  if (device_index < 0 || device_index >= count) return tsr::kInvalidArgument;
  cudaError_t e = cudaSetDevice(device_index);
  if (e != cudaSuccess) return map_cuda(e);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device_index);
  if (e != cudaSuccess) return map_cuda(e);
  if (prop.major != 10) {
    // The kernels are built for sm_100a only; there is no other code path.
    std::fprintf(stderr, "tessera_b200: device %d is sm_%d%d, this library holds sm_100a code only\n",
                 device_index, prop.major, prop.minor);
    return tsr::kUnsupportedFeature;
  }
  auto* ctx = new tsr_context();
  ctx->device = device_index;
  if (borrow) {
    ctx->stream = borrowed;
  } else {
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      delete ctx;
      return map_cuda(e);
    }
    ctx->owns_stream = true;
  }
  e = cudaHostAlloc(reinterpret_cast<void**>(&ctx->stage), kStageWindow * kStageWindows,
                    cudaHostAllocDefault);
  if (e != cudaSuccess) {
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return map_cuda(e);
  }
  for (int i = 0; i < kStageWindows; ++i)
    cudaEventCreateWithFlags(&ctx->stage_done[i], cudaEventDisableTiming);
  // Split-K scratch of the merged launches, held for the life of the context so
  // that no launch ever allocates (graphs keep its address).
  void* scratch = nullptr;
  e = cudaMalloc(&scratch, kScratchFloats * 4 + kScratchTickets * 4);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(ctx->stage);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return map_cuda(e);
  }
  ctx->scratch.part = static_cast<float*>(scratch);
  ctx->scratch.part_floats = kScratchFloats;
  ctx->scratch.tickets = reinterpret_cast<unsigned int*>(ctx->scratch.part + kScratchFloats);
  ctx->scratch.ntickets = kScratchTickets;
  cudaMemset(ctx->scratch.tickets, 0, kScratchTickets * 4);
  publish_error_word(device_index);
  if (const unsigned int* word = host_error_word()) ctx->seen_error_word = *reinterpret_cast<const volatile unsigned int*>(word);
  // Keep freed pool memory cached: a mid-step scratch growth must not pay
  // for a device allocation twice.
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device_index) == cudaSuccess) {
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  *out = ctx;
  return tsr::kOk;
}

int tsr_create(int device_index, tsr_context** out) {
  return create_common(device_index, nullptr, false, out);
}

int tsr_create_on_stream(int device_index, void* cuda_stream, tsr_context** out) {
  return create_common(device_index, static_cast<cudaStream_t>(cuda_stream), true, out);
}

void tsr_destroy(tsr_context* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  tsr::flush_pending(ctx);
  cudaStreamSynchronize(ctx->stream);
  for (auto& g : ctx->graphs)
    if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  cudaFree(ctx->scratch.part);
  for (int i = 0; i < kStageWindows; ++i) cudaEventDestroy(ctx->stage_done[i]);
  cudaFreeHost(ctx->stage);
  if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

int tsr_context_device(const tsr_context* ctx) { return ctx ? ctx->device : -1; }
void* tsr_context_stream(const tsr_context* ctx) { return ctx ? ctx->stream : nullptr; }
const char* tsr_last_error(const tsr_context* ctx) { return ctx ? ctx->error.c_str() : "no context"; }

int tsr_memory_info(tsr_context* ctx, uint64_t* total_bytes, uint64_t* free_bytes) {
  if (!ctx || !total_bytes || !free_bytes) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  size_t f = 0, t = 0;
  const cudaError_t e = cudaMemGetInfo(&f, &t);
  if (e != cudaSuccess) return ctx->fail(e, "cudaMemGetInfo");
  *total_bytes = t;
  *free_bytes = f;
  return tsr::kOk;
}

int tsr_alloc(tsr_context* ctx, size_t bytes, int kind, void** handle, void** host_map) {
  if (!ctx || !handle || bytes == 0) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  *handle = nullptr;
  if (host_map) *host_map = nullptr;
  if (kind == TSR_MEM_DEVICE) {
    // Stream-ordered pool allocation: no device-wide synchronisation.
    const cudaError_t e = cudaMallocAsync(handle, bytes, ctx->stream);
    if (e != cudaSuccess) return ctx->fail(e, "cudaMallocAsync");
    return tsr::kOk;
  }
  if (kind == TSR_MEM_HOST_VISIBLE) {
    const cudaError_t e = cudaHostAlloc(handle, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return ctx->fail(e, "cudaHostAlloc");
    if (host_map) *host_map = *handle;
    return tsr::kOk;
  }
  return tsr::kInvalidArgument;
}

int tsr_free(tsr_context* ctx, int kind, void* handle) {
  if (!ctx) return tsr::kInvalidArgument;
  if (!handle) return tsr::kOk;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;  // a queued launch may use the buffer
  cudaError_t e;
  if (kind == TSR_MEM_DEVICE) {
    e = cudaFreeAsync(handle, ctx->stream);
  } else {
    cudaStreamSynchronize(ctx->stream);
    e = cudaFreeHost(handle);
  }
  return e == cudaSuccess ? tsr::kOk : ctx->fail(e, "free");
}

int tsr_copy_h2d(tsr_context* ctx, void* dst, size_t dst_offset, const void* src, size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return tsr::kInvalidArgument;
  if (bytes == 0) return tsr::kOk;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  std::lock_guard<std::mutex> lock(ctx->mutex);
  auto* d = static_cast<unsigned char*>(dst) + dst_offset;
  const auto* h = static_cast<const unsigned char*>(src);
  for (size_t done = 0; done < bytes;) {
    const size_t n = bytes - done < kStageWindow ? bytes - done : kStageWindow;
    int wi;
    unsigned char* win = ctx->window(&wi);
    std::memcpy(win, h + done, n);
    cudaError_t e = cudaMemcpyAsync(d + done, win, n, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return ctx->fail(e, "cudaMemcpyAsync(h2d)");
    cudaEventRecord(ctx->stage_done[wi], ctx->stream);
    ctx->stage_busy[wi] = true;
    done += n;
  }
  return tsr::kOk;
}

int tsr_copy_d2h(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return tsr::kInvalidArgument;
  if (bytes == 0) return tsr::kOk;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  std::lock_guard<std::mutex> lock(ctx->mutex);
  const auto* d = static_cast<const unsigned char*>(src) + src_offset;
  auto* h = static_cast<unsigned char*>(dst);
  for (size_t done = 0; done < bytes;) {
    // Up to all windows in flight, then drain them in order.
    size_t offs[kStageWindows], lens[kStageWindows];
    unsigned char* wins[kStageWindows];
    int used = 0;
    while (used < kStageWindows && done < bytes) {
      const size_t n = bytes - done < kStageWindow ? bytes - done : kStageWindow;
      int wi;
      wins[used] = ctx->window(&wi);
      cudaError_t e = cudaMemcpyAsync(wins[used], d + done, n, cudaMemcpyDeviceToHost, ctx->stream);
      if (e != cudaSuccess) return ctx->fail(e, "cudaMemcpyAsync(d2h)");
      offs[used] = done;
      lens[used] = n;
      done += n;
      ++used;
    }
    const cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return ctx->fail(e, "cudaStreamSynchronize(d2h)");
    for (int i = 0; i < used; ++i) std::memcpy(h + offs[i], wins[i], lens[i]);
  }
  return tsr::kOk;
}

int tsr_copy_d2d(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t dst_offset,
                 size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return tsr::kInvalidArgument;
  if (bytes == 0) return tsr::kOk;
  if (int s = ctx->select()) return s;
  if (ctx->deferred && bytes <= tsr::kQueuedCopyLimit) return tsr::queue_copy(ctx, src, src_offset, dst, dst_offset, bytes);
  if (int s = tsr::flush_pending(ctx)) return s;
  const cudaError_t e = cudaMemcpyAsync(static_cast<unsigned char*>(dst) + dst_offset,
                                        static_cast<const unsigned char*>(src) + src_offset, bytes,
                                        cudaMemcpyDeviceToDevice, ctx->stream);
  return e == cudaSuccess ? tsr::kOk : ctx->fail(e, "cudaMemcpyAsync(d2d)");
}

int tsr_copy_peer(tsr_context* ctx, void* dst, int src_device, const void* src, size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return tsr::kInvalidArgument;
  if (bytes == 0) return tsr::kOk;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  if (src_device != ctx->device && src_device >= 0 && src_device < 64 &&
      !ctx->peer_enabled[src_device]) {
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, ctx->device, src_device) == cudaSuccess && can) {
      const cudaError_t e = cudaDeviceEnablePeerAccess(src_device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
        return ctx->fail(e, "cudaDeviceEnablePeerAccess");
      cudaGetLastError();
    }
    ctx->peer_enabled[src_device] = true;  // cudaMemcpyPeer stages by itself when no peer path
  }
  cudaError_t e = cudaMemcpyPeerAsync(dst, ctx->device, src, src_device, bytes, ctx->stream);
  if (e != cudaSuccess) return ctx->fail(e, "cudaMemcpyPeerAsync");
  e = cudaStreamSynchronize(ctx->stream);
  return e == cudaSuccess ? tsr::kOk : ctx->fail(e, "cudaStreamSynchronize(peer)");
}

int tsr_synchronize(tsr_context* ctx) {
  if (!ctx) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  const cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return ctx->fail(e, "cudaStreamSynchronize");
  // A kernel whose bounded wait ran out has left wrong results behind: it raised the
  // host-visible error word.  Only then are the per-file counters worth a copy each.
  const unsigned int* word = host_error_word();
  const unsigned int raised = word ? *reinterpret_cast<const volatile unsigned int*>(word) : 0u;
  if (word == nullptr || raised != 0u) {
    unsigned int timeouts = 0, umma = 0, q6k = 0, f16 = 0, f8 = 0;
    tsr::umma_wait_timeouts(&umma);
    tsr::umma_f8_wait_timeouts(&f8);
    tsr::staged_q6k_wait_timeouts(&q6k);
    tsr::staged_f16_wait_timeouts(&f16);
    if (tsr::staged_wait_timeouts(&timeouts) == tsr::kOk && (timeouts += umma + q6k + f16 + f8) != ctx->seen_timeouts) {
      ctx->seen_timeouts = timeouts;
      ctx->error = "a staged kernel gave up waiting for a TMA copy";
      return tsr::kDeviceError;
    }
  }
  return tsr::kOk;
}

int tsr_set_deferred(tsr_context* ctx, int on) {
  if (!ctx) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  ctx->deferred = on != 0;
  ctx->use_graphs = on != 2;
  ctx->fold_elementwise = on != 3;
  return tsr::kOk;
}

int tsr_flush(tsr_context* ctx) {
  if (!ctx) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  return tsr::flush_pending(ctx);
}

int tsr_launch_stats(tsr_context* ctx, uint64_t* api_launches, uint64_t* device_kernels, uint64_t* graph_launches) {
  if (!ctx) return tsr::kInvalidArgument;
  if (api_launches) *api_launches = ctx->stats.api_launches;
  if (device_kernels) *device_kernels = ctx->stats.device_kernels;
  if (graph_launches) *graph_launches = ctx->stats.graph_launches;
  return tsr::kOk;
}

int tsr_tp_bind(tsr_context* ctx, tsr_tp_comm* comm) {
  if (!ctx) return tsr::kInvalidArgument;
  if (int s = ctx->select()) return s;
  if (int s = tsr::flush_pending(ctx)) return s;
  if (comm != nullptr && tsr::tp_device_of(comm) != ctx->device) return tsr::kInvalidArgument;
  ctx->tp = comm;
  return tsr::kOk;
}

}  // extern "C"
