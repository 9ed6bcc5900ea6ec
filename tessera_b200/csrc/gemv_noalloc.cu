// Split-K Q4_K projection that never allocates device memory.
//
// Some hosts cannot let a projection call allocate: an engine that has
// budgeted every byte of device memory before it starts serving (the weights,
// the KV cache and its scratch are sized from the free-memory figure at load
// time, so a later cudaMalloc can fail or push it over), or a caller that sits
// inside a latency-critical decode loop where cudaMalloc's device-wide
// synchronisation would stall every stream.  The ordinary split-K path needs
// a partial-sum buffer of split*m*n floats that such a caller would have to
// allocate; this entry point keeps that buffer in a fixed array that is part
// of the library image instead.
#include <cuda_runtime.h>

#include <mutex>

#include "launch.h"
#include "tessera_b200.h"

namespace {

// Partial sums of the split-K chunks: region y holds the m*n outputs of
// chunk y.  4 MiB per GPU that loads the library, held until the process ends.
constexpr unsigned long long kScratchFloats = 1ull << 20;
static __device__ __align__(256) float g_split_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_address[kMaxDevices] = {};

// The array's name is only a host-side stand-in; the device address has to be
// asked for, once per device, with that device current.
int scratch_for_current_device(float** out) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return tsr::kDeviceError;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_split_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return tsr::kDeviceError;
    }
    g_scratch_address[device] = static_cast<float*>(ptr);
  }
  *out = g_scratch_address[device];
  return tsr::kOk;
}

}  // namespace

extern "C" {

uint64_t tsr_gemm_q4k_noalloc_max_outputs(void) { return kScratchFloats; }

int tsr_gemm_q4k_noalloc(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                         void* stream) {
  if (!a || !w || !c || m == 0 || n == 0 || k == 0 || k % 256 != 0 || m > 0x7FFFFFFFull ||
      n > 0x7FFFFFFFull || k > 0x7FFFFFFFull)
    return tsr::kInvalidArgument;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(c)) & 15u)
    return tsr::kInvalidArgument;
  const uint64_t outputs = m * n;
  if (outputs > kScratchFloats) return tsr::kInvalidArgument;  // beyond the fixed scratch
  // Largest split of at most 8 that divides the block count and still fits.
  const uint64_t blocks = k / 256;
  uint64_t split = 8;
  while (split > 1 && (blocks % split != 0 || split * outputs > kScratchFloats)) --split;
  float* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  // Every element of the regions in use is overwritten by the projection, so
  // nothing has to be cleared between calls.
  // A batch with no usable split goes straight to c.  Either way no path below
  // may allocate: the batched tile is told to do without its activation scratch.
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (split == 1) return tsr::gemm_q4k_dispatch(a, w, c, m, n, k, 1, st, false);
  if (int rc = tsr::gemm_q4k_dispatch(a, w, scratch, m, n, k, split, st, false)) return rc;
  return tsr_gemm_vec_reduce(scratch, c, outputs, split, stream);
}

}  // extern "C"
