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

// Staged tensor-pipe kernels (gemv_mma.cu).  kUnsupportedFeature means the
// shape is outside their range and the caller uses the general family.
int staged_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    uint64_t split, cudaStream_t st);
// Number of bounded device waits that gave up since the library was loaded.
int staged_wait_timeouts(unsigned int* count);

// tcgen05/TMEM tile for small batches (gemm_umma.cu).  fmt: 0 Q4_K, 1 Q6_K,
// 2 MXFP4, 3 FP8.  kUnsupportedFeature when the shape is outside its range.
int umma_gemm(int fmt, const float* a, const void* w, const float* scale, float* c, uint64_t m,
              uint64_t n, uint64_t k, cudaStream_t st);
int umma_wait_timeouts(unsigned int* count);

}  // namespace tsr
