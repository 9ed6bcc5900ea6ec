// tessera::Backend implemented over the sm_100a C ABI (include/tessera_b200.h).
//
// This is the drop-in seam of the reference: a third backend beside
// src/backends/vulkan and src/backends/rocm.  It is compiled against the
// reference's own headers (include/tessera/backend.hpp) and linked into the
// engine in place of those backends; CreateBackend() and ListGpuNames()
// (backend.hpp:1062-1071) are the only symbols the core needs.  The ROCm
// backend (src/backends/rocm/rocm_backend.cpp) is the behavioural model:
// one stream, stream-ordered launches, blocking device-to-host copies,
// UnsupportedFeature for ids this backend does not implement so that the
// core's callers fall back (src/core/decode_internal.hpp:1297-1323).
//
// No computation happens in this file; every method forwards to the C ABI.
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <expected>
#include <memory>
#include <span>
#include <string>
#include <string_view>
#include <vector>

#include "tessera/backend.hpp"
#include "tessera_b200.h"

namespace tessera {
namespace {

StatusCode FromCode(int code) {
  switch (code) {
    case TSR_OK: return StatusCode::Ok;
    case TSR_INVALID_ARGUMENT: return StatusCode::InvalidArgument;
    case TSR_UNSUPPORTED_FEATURE: return StatusCode::UnsupportedFeature;
    case TSR_OUT_OF_MEMORY: return StatusCode::OutOfMemory;
    default: return StatusCode::DeviceError;
  }
}

class CudaBackend final : public Backend {
 public:
  ~CudaBackend() override {
    if (ctx_ != nullptr) {
      tsr_destroy(ctx_);
    }
  }

  [[nodiscard]] std::string_view Name() const override { return "cuda"; }
  [[nodiscard]] std::string_view DeviceName() const override { return device_name_; }

  [[nodiscard]] DeviceMemoryInfo MemoryInfo() const override {
    DeviceMemoryInfo info;
    if (ctx_ != nullptr) {
      std::uint64_t total = 0, free_bytes = 0;
      if (tsr_memory_info(ctx_, &total, &free_bytes) == TSR_OK) {
        info.total_bytes = total;
        info.free_bytes = free_bytes;
      }
    }
    return info;
  }

  std::expected<void, StatusCode> Init() override {
    if (ctx_ != nullptr) {
      return {};
    }
    const int code = tsr_create(device_index_, &ctx_);
    if (code != TSR_OK) {
      LogError("cuda backend: no usable sm_100a device at index " +
               std::to_string(device_index_));
      return std::unexpected(FromCode(code));
    }
    // Launches queue until the next copy or synchronisation, are merged where
    // the kernels allow it and replayed as a CUDA graph when they repeat: the
    // core issues hundreds of launches per token (rocm_backend.cpp:697-699).
    // TESSERA_CUDA_DEFERRED=0 issues every launch at once, =2 merges without graphs.
    int deferred = 1;
    if (const char* v = std::getenv("TESSERA_CUDA_DEFERRED")) {
      deferred = std::atoi(v);
    }
    tsr_set_deferred(ctx_, deferred);
    char name[256] = {};
    tsr_device_name(device_index_, name, sizeof(name));
    device_name_ = name;
    LogInfo("cuda backend: device " + std::to_string(device_index_) + " " +
            device_name_);
    return {};
  }

  std::expected<std::unique_ptr<Buffer>, StatusCode> AllocateBuffer(
      std::size_t bytes, MemoryKind kind) override {
    if (bytes == 0 || ctx_ == nullptr) {
      return std::unexpected(bytes == 0 ? StatusCode::InvalidArgument
                                        : StatusCode::DeviceError);
    }
    void* handle = nullptr;
    void* host_map = nullptr;
    const int code =
        tsr_alloc(ctx_, bytes, static_cast<int>(kind), &handle, &host_map);
    if (code != TSR_OK) {
      return Fail<std::unique_ptr<Buffer>>(code, "AllocateBuffer");
    }
    return AdoptBuffer(handle, bytes, kind, host_map);
  }

  void FreeBuffer(MemoryKind kind, void* handle) override {
    if (ctx_ != nullptr) {
      tsr_free(ctx_, static_cast<int>(kind), handle);
    }
  }

  std::expected<void, StatusCode> CopyH2D(
      Buffer& dst, std::span<const std::byte> src) override {
    return CopyH2DAt(dst, 0, src);
  }

  std::expected<void, StatusCode> CopyH2DAt(
      Buffer& dst, std::size_t offset,
      std::span<const std::byte> src) override {
    if (offset > dst.Size() || src.size() > dst.Size() - offset) {
      return std::unexpected(StatusCode::InvalidArgument);
    }
    return Done(tsr_copy_h2d(ctx_, dst.Handle(), offset, src.data(), src.size()),
                "CopyH2D");
  }

  std::expected<void, StatusCode> CopyD2H(const Buffer& src, std::byte* dst,
                                          std::size_t bytes) override {
    return CopyD2HAt(src, 0, dst, bytes);
  }

  std::expected<void, StatusCode> CopyD2HAt(const Buffer& src,
                                            std::size_t offset, std::byte* dst,
                                            std::size_t bytes) override {
    if (offset > src.Size() || bytes > src.Size() - offset) {
      return std::unexpected(StatusCode::InvalidArgument);
    }
    return Done(tsr_copy_d2h(ctx_, src.Handle(), offset, dst, bytes), "CopyD2H");
  }

  std::expected<void, StatusCode> CopyD2D(const Buffer& src,
                                          std::size_t src_offset, Buffer& dst,
                                          std::size_t dst_offset,
                                          std::size_t bytes) override {
    if (src_offset > src.Size() || bytes > src.Size() - src_offset ||
        dst_offset > dst.Size() || bytes > dst.Size() - dst_offset) {
      return std::unexpected(StatusCode::InvalidArgument);
    }
    return Done(tsr_copy_d2d(ctx_, src.Handle(), src_offset, dst.Handle(),
                             dst_offset, bytes),
                "CopyD2D");
  }

  std::expected<void, StatusCode> CopyPeerFrom(Buffer& dst, const Buffer& src,
                                               std::size_t bytes) override {
    if (bytes == 0) {
      return {};
    }
    if (bytes > dst.Size() || bytes > src.Size()) {
      return std::unexpected(StatusCode::InvalidArgument);
    }
    if (src.Owner().Name() != "cuda") {
      return Backend::CopyPeerFrom(dst, src, bytes);
    }
    // The source must be quiescent before the peer read (backend.hpp:1039-1045).
    src.Owner().Synchronize();
    return Done(tsr_copy_peer(ctx_, dst.Handle(), src.Owner().DeviceIndex(),
                              src.Handle(), bytes),
                "CopyPeerFrom");
  }

  std::expected<std::unique_ptr<Kernel>, StatusCode> LoadKernel(
      std::string_view name, std::span<const std::byte> code) override {
    if (!code.empty()) {
      LogError("kernel '" + std::string(name) +
               "': compiled kernel modules are not supported on cuda; use a "
               "built-in kernel id");
      return std::unexpected(StatusCode::UnsupportedFeature);
    }
    const int index = tsr_kernel_lookup(std::string(name).c_str());
    if (index < 0) {
      // Quiet: the core probes optional ids and falls back on this status.
      return std::unexpected(StatusCode::UnsupportedFeature);
    }
    return AdoptKernel(
        reinterpret_cast<void*>(static_cast<std::uintptr_t>(index) + 1), name);
  }

  void FreeKernel(void* handle) override { (void)handle; }

  std::expected<void, StatusCode> LaunchKernel(
      const Kernel& kernel, const KernelLaunch& launch) override {
    if (ctx_ == nullptr) {
      return std::unexpected(StatusCode::DeviceError);
    }
    if (const StatusCode invalid = ValidateLaunch(launch);
        invalid != StatusCode::Ok) {
      return std::unexpected(invalid);
    }
    if (const StatusCode missing = CheckBuiltInArgs(kernel, launch);
        missing != StatusCode::Ok) {
      return std::unexpected(missing);
    }
    const void* buffers[kMaxBoundBuffers];
    std::size_t sizes[kMaxBoundBuffers];
    std::size_t count = 0;
    for (const Buffer* buffer : launch.buffers) {
      if (buffer == nullptr) {
        return std::unexpected(StatusCode::InvalidArgument);
      }
      buffers[count] = buffer->Handle();
      sizes[count] = buffer->Size();
      ++count;
    }
    const std::uint32_t grid[3] = {launch.grid_x, launch.grid_y, launch.grid_z};
    const std::uint32_t block[3] = {launch.block_x, launch.block_y,
                                    launch.block_z};
    const int index = static_cast<int>(
        reinterpret_cast<std::uintptr_t>(kernel.Handle()) - 1);
    const int code = tsr_launch(ctx_, index, grid, block, buffers, sizes,
                                static_cast<int>(count), launch.scalars.data(),
                                static_cast<int>(launch.scalars.size()));
    if (code != TSR_OK) {
      LogError("kernel " + std::string(kernel.Id()) + " launch failed (" +
               std::string(ToString(FromCode(code))) + ")");
      return std::unexpected(FromCode(code));
    }
    return {};
  }

  void Synchronize() override {
    if (ctx_ != nullptr && tsr_synchronize(ctx_) != TSR_OK) {
      LogError(std::string("cuda synchronize failed: ") + tsr_last_error(ctx_));
    }
  }

 private:
  template <typename T>
  std::expected<T, StatusCode> Fail(int code, const char* what) {
    LogError(std::string("cuda ") + what + ": " +
             (ctx_ != nullptr ? tsr_last_error(ctx_) : "no context"));
    return std::unexpected(FromCode(code));
  }
  std::expected<void, StatusCode> Done(int code, const char* what) {
    if (code == TSR_OK) {
      return {};
    }
    return Fail<void>(code, what);
  }

  tsr_context* ctx_ = nullptr;
  std::string device_name_;
};

}  // namespace

std::unique_ptr<Backend> CreateBackend() {
  return std::make_unique<CudaBackend>();
}

std::expected<std::vector<std::string>, StatusCode> ListGpuNames() {
  int count = 0;
  if (tsr_device_count(&count) != TSR_OK || count == 0) {
    return std::unexpected(StatusCode::DeviceError);
  }
  std::vector<std::string> names;
  for (int i = 0; i < count; ++i) {
    char name[256] = {};
    if (tsr_device_name(i, name, sizeof(name)) != TSR_OK) {
      return std::unexpected(StatusCode::DeviceError);
    }
    names.emplace_back(name);
  }
  return names;
}

}  // namespace tessera
