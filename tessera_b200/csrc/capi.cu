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

#include "launch.h"
#include "tessera_b200.h"

namespace {

constexpr size_t kStageWindow = 4u << 20;  // bytes per pinned staging window
constexpr int kStageWindows = 8;

int map_cuda(cudaError_t e) {
  if (e == cudaSuccess) return tsr::kOk;
  if (e == cudaErrorMemoryAllocation) return tsr::kOutOfMemory;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidDevice) return tsr::kInvalidArgument;
  return tsr::kDeviceError;
}

}  // namespace

struct tsr_context {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  std::string error;
  // Pinned staging ring for host<->device copies: a window is reused only
  // after the copy that read or wrote it has completed (event guard).
  unsigned char* stage = nullptr;
  cudaEvent_t stage_done[kStageWindows] = {};
  bool stage_busy[kStageWindows] = {};
  int stage_next = 0;
  bool peer_enabled[64] = {};
  unsigned int seen_timeouts = 0;
  std::mutex mutex;

  int fail(cudaError_t e, const char* what) {
    char buf[256];
    std::snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    error = buf;
    return map_cuda(e);
  }
  int select() {
    // The current device is per host thread and the reference drives one
    // backend from different threads over time (a fresh thread per
    // tensor-parallel step): re-select on every entry.
    // cudaSetDevice on the already-current device is a cheap no-op; no cache
    // is kept because other entry points of the library also switch devices.
    const cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(e, "cudaSetDevice");
    return tsr::kOk;
  }
  unsigned char* window(int* index) {
    const int i = stage_next;
    stage_next = (stage_next + 1) % kStageWindows;
    if (stage_busy[i]) {
      cudaEventSynchronize(stage_done[i]);
      stage_busy[i] = false;
    }
    *index = i;
    return stage + static_cast<size_t>(i) * kStageWindow;
  }
};

namespace tsr {

// Last output range written by a launch of this library, per stream.
bool pdl_allowed(cudaStream_t stream, const void* read_ptr, size_t read_bytes, const void* out_ptr,
                 size_t out_bytes) {
  static const bool enabled = [] {
    const char* v = std::getenv("TSR_PDL");
    return v == nullptr || std::atoi(v) != 0;
  }();
  struct Last {
    cudaStream_t stream;
    const unsigned char* ptr;
    size_t bytes;
  };
  static std::mutex mutex;
  static Last table[16] = {};
  std::lock_guard<std::mutex> lock(mutex);
  Last* slot = nullptr;
  for (Last& l : table)
    if (l.ptr != nullptr && l.stream == stream) slot = &l;
  bool ok = enabled;
  if (slot != nullptr) {
    const auto* r = static_cast<const unsigned char*>(read_ptr);
    if (r < slot->ptr + slot->bytes && slot->ptr < r + read_bytes) ok = false;  // previous output is our weight
  }
  if (slot == nullptr) {
    static int next = 0;
    slot = &table[next];
    next = (next + 1) % 16;
  }
  *slot = Last{stream, static_cast<const unsigned char*>(out_ptr), out_bytes};
  return ok;
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
  cudaStreamSynchronize(ctx->stream);
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
  const cudaError_t e = cudaMemcpyAsync(static_cast<unsigned char*>(dst) + dst_offset,
                                        static_cast<const unsigned char*>(src) + src_offset, bytes,
                                        cudaMemcpyDeviceToDevice, ctx->stream);
  return e == cudaSuccess ? tsr::kOk : ctx->fail(e, "cudaMemcpyAsync(d2d)");
}

int tsr_copy_peer(tsr_context* ctx, void* dst, int src_device, const void* src, size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return tsr::kInvalidArgument;
  if (bytes == 0) return tsr::kOk;
  if (int s = ctx->select()) return s;
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
  const cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return ctx->fail(e, "cudaStreamSynchronize");
  // A staged kernel whose bounded wait ran out has left wrong results behind.
  unsigned int timeouts = 0, umma = 0, q6k = 0, f16 = 0;
  tsr::umma_wait_timeouts(&umma);
  tsr::staged_q6k_wait_timeouts(&q6k);
  tsr::staged_f16_wait_timeouts(&f16);
  if (tsr::staged_wait_timeouts(&timeouts) == tsr::kOk && (timeouts += umma + q6k + f16) != ctx->seen_timeouts) {
    ctx->seen_timeouts = timeouts;
    ctx->error = "a staged kernel gave up waiting for a TMA copy";
    return tsr::kDeviceError;
  }
  return tsr::kOk;
}

}  // extern "C"
