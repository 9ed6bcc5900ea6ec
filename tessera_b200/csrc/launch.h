// Internal launcher prototypes shared by the .cu files of the library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tsr {

// Status values equal tessera::StatusCode (include/tessera/types.hpp:38-48).
constexpr int kOk = 0;
constexpr int kInvalidArgument = 1;
constexpr int kUnsupportedFeature = 4;
constexpr int kOutOfMemory = 5;
constexpr int kDeviceError = 6;

// Maps the pending launch error (cudaGetLastError) to a status.
inline int check_launch() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return kOk;
  if (e == cudaErrorMemoryAllocation) return kOutOfMemory;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidConfiguration) return kInvalidArgument;
  return kDeviceError;
}

// ---- programmatic dependent launch -----------------------------------------
// A kernel launched with `pdl` set may begin while the previous kernel of the
// stream is still running; it must execute pdl_wait() before it touches
// anything that kernel wrote (or writes anything that kernel reads), and calls
// pdl_trigger() after that wait so that at most two kernels ever overlap.
// Before the wait the staged kernels only prefetch weights, so the launcher
// drops the attribute when the previous launch of this library on the stream
// wrote into the weight range (pdl_allowed).
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster` consecutive CTAs along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, bool pdl, unsigned cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned count = 0;
  if (cluster > 1) {
    attr[count].id = cudaLaunchAttributeClusterDimension;
    attr[count].val.clusterDim.x = cluster;
    attr[count].val.clusterDim.y = 1;
    attr[count].val.clusterDim.z = 1;
    ++count;
  }
  if (pdl) {
    attr[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  cfg.attrs = attr;
  cfg.numAttrs = count;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
// Raises the dynamic shared-memory limit of `kernel` on the current device, once per
// (kernel, device): the attribute belongs to the device, and one process may drive
// several GPUs (the reference runs its tensor-parallel ranks as threads).
int allow_dynamic_smem(const void* kernel, int bytes);

// True when a kernel that reads [read_ptr, +read_bytes) before its pdl_wait()
// may overlap the previous launch on `stream`; records [out_ptr, +out_bytes) as
// the range this launch writes.
bool pdl_allowed(cudaStream_t stream, const void* read_ptr, size_t read_bytes, const void* out_ptr,
                 size_t out_bytes);

// General warp-per-row family (gemv_rows.cu).
int rows_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                  uint64_t split, cudaStream_t st);
int rows_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                  uint64_t split, cudaStream_t st);
int rows_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    cudaStream_t st);
int rows_gemm_fp8(const float* a, const void* w, const float* s, float* c, uint64_t m, uint64_t n,
                  uint64_t k, cudaStream_t st);
int rows_gemm_w4a8(const void* a8, const void* w, const float* as, const void* wref, float* c,
                   uint64_t m, uint64_t n, uint64_t k, uint64_t split, cudaStream_t st);

// Staged tensor-pipe kernels (gemv_mma.cu, gemv_q6k_mma.cu, gemv_f16_mma.cu).  kUnsupportedFeature means the
// shape is outside their range and the caller uses the general family.
int staged_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    uint64_t split, cudaStream_t st);
int staged_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    uint64_t split, cudaStream_t st);
int staged_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                      cudaStream_t st);
int staged_gemm_fp8(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n,
                    uint64_t k, cudaStream_t st);
// Number of bounded device waits that gave up since the library was loaded.
int staged_wait_timeouts(unsigned int* count);
int staged_q6k_wait_timeouts(unsigned int* count);
int staged_f16_wait_timeouts(unsigned int* count);

// tcgen05/TMEM tile for small batches (gemm_umma.cu).  fmt: 0 Q4_K, 1 Q6_K,
// 2 MXFP4, 3 FP8.  kUnsupportedFeature when the shape is outside its range.
int umma_gemm(int fmt, const float* a, const void* w, const float* scale, float* c, uint64_t m,
              uint64_t n, uint64_t k, cudaStream_t st);
int umma_wait_timeouts(unsigned int* count);

}  // namespace tsr
