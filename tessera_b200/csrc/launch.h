// Internal launcher prototypes shared by the .cu files of the library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace tsr {

// Status values equal tessera::StatusCode (include/tessera/types.hpp:38-48).
constexpr int kOk = 0;
constexpr int kInvalidArgument = 1;
constexpr int kUnsupportedFeature = 4;
constexpr int kOutOfMemory = 5;
constexpr int kDeviceError = 6;

// Kernel launches this library has issued in this process (every launcher ends with
// check_launch(), which counts); a captured graph replays as many as were captured.
inline std::atomic<uint64_t>& launch_counter() {
  static std::atomic<uint64_t> count{0};
  return count;
}

// Maps the pending launch error (cudaGetLastError) to a status.
inline int check_launch() {
  launch_counter().fetch_add(1, std::memory_order_relaxed);
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

// The same with thread-block clusters of `cluster_y` consecutive CTAs along y.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster_y(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, bool pdl, unsigned cluster_y, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned count = 0;
  if (cluster_y > 1) {
    attr[count].id = cudaLaunchAttributeClusterDimension;
    attr[count].val.clusterDim.x = 1;
    attr[count].val.clusterDim.y = cluster_y;
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

// Multi-range form of pdl_allowed (a launch over several weight tensors): true when none of the
// `reads` ranges overlaps a range the previous launch of this library on `stream` wrote; records
// `writes` as what this launch writes (more than twelve ranges: the next launch is refused).
// Invariant the staged kernels rely on: before its pdl_wait() a kernel reads weight bytes only, and
// a weight range is only ever written by a copy (a stream-ordered memcpy is never overlapped) or by
// a launch of this library that registers its output here.  A foreign kernel that writes weights
// must be followed by a stream synchronisation or by a launch without the programmatic attribute.
bool pdl_allowed_ranges(cudaStream_t stream, const void* const* reads, const size_t* read_bytes, int nreads,
                        const void* const* writes, const size_t* write_bytes, int nwrites);

// True when a kernel that reads [read_ptr, +read_bytes) before its pdl_wait()
// may overlap the previous launch on `stream`; records [out_ptr, +out_bytes) as
// the range this launch writes.
bool pdl_allowed(cudaStream_t stream, const void* read_ptr, size_t read_bytes, const void* out_ptr,
                 size_t out_bytes);

// ---- tensor-parallel tail and multi-target launches ---------------------------
constexpr int kMaxWorld = 8;
#ifndef TSR_MAX_GROUP
#define TSR_MAX_GROUP 4
#endif
constexpr int kMaxGroup = TSR_MAX_GROUP;  // weight tensors one staged launch can serve
// What a kernel needs to finish with the sum over tensor-parallel ranks
// (tp_device.cuh explains the protocol and the memory behind the pointers).
struct TpTail {
  int world;  // 1: no collective
  int rank;
  unsigned long long capacity;  // floats per slot
  float* slots[kMaxWorld];      // slot memory of every rank (this rank's own included)
  unsigned int* state;          // this rank's state words
};
// One weight tensor of a multi-target launch: C[m, n] = A . dq(W)^T.
struct GroupTarget {
  const void* w;
  float* c;
  uint64_t n;
  // add_out[e] = add_src[e] + C[e] written besides C (the reference's "add" after a projection,
  // include/tessera/backend.hpp:255-256); null: none
  const float* add_src = nullptr;
  float* add_out = nullptr;
};
// What a staged launch does around its projection: an elementwise step folded into the
// activation staging, and bf16 storage of the activations and outputs.
// (kProRmsNormLate is chosen by the launchers themselves: the same result, the gain applied to the
// sums instead of the activations, staged_common.cuh)
enum : int { kProNone = 0, kProSiluMul = 1, kProRmsNorm = 2, kProRmsNormLate = 3 };
struct Prologue {
  int kind;            // kProSiluMul: A = silu(a) * other; kProRmsNorm: A = a / sqrt(mean(a^2) + eps) * other
  const float* other;  // up vector [m][k] / norm weights [k]
  float* out;          // receives A ([m][k]); may be null
  float eps;
  // a points to bf16 values (read as fp32 with a zero low half) / every c points to bf16
  // storage and receives the sums rounded to nearest even (RoundBf16Ref,
  // src/core/numerics/quant.cpp:231-243 of the reference).  Not combined with `kind` or an add.
  bool bf16_in = false;
  bool bf16_out = false;
};
// Device scratch of a context for launches that split k among CTAs and add the
// chunks themselves: partial tiles and one arrival counter per tile (zero at rest).
struct FusedScratch {
  float* part;
  size_t part_floats;
  unsigned int* tickets;
  size_t ntickets;
};
// Multi-target staged launches (gemv_mma.cu, gemv_q6k_mma.cu): up to four weight tensors that
// share a, m and k.  caller_split >= 1: chunk y of k goes to region y of each target;
// caller_split == 0: the launch picks its own split and adds the chunks (and, with `tp`, the ranks).
// `pro` (null: none) and the targets' add_src/add_out need caller_split == 0.
int staged_group_q4k(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                     const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro = nullptr);
int staged_group_q6k(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                     const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro = nullptr);

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
              uint64_t n, uint64_t k, cudaStream_t st, bool allow_scratch = true);
// What tsr_gemm_q4k runs after its argument checks.  allow_scratch false keeps every path
// away from device allocations (the allocation-free entry point uses it).
int gemm_q4k_dispatch(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                      uint64_t split, cudaStream_t st, bool allow_scratch);
int umma_wait_timeouts(unsigned int* count);
// Device scratch of a (device, stream) pair, grown on demand from the stream-ordered pool and
// kept until exit (a captured graph may hold the pointer).  Null when the stream is being
// captured and no large enough buffer exists yet.  Work on one stream uses it in stream order.
unsigned char* stream_scratch(cudaStream_t st, size_t bytes, int slot = 0);
// bf16 <-> fp32 copies on the stream (elementwise.cu); the fp32 -> bf16 direction rounds to nearest even
int convert_bf16_to_f32(const void* src, float* dst, uint64_t n, cudaStream_t st);
int convert_f32_to_bf16(const float* src, void* dst, uint64_t n, cudaStream_t st);
// tcgen05 tile over 8-bit weights read straight from shared memory (gemm_f8_umma.cu): FP8
// weights, 2..21 activation rows.  kUnsupportedFeature when the shape is outside its range.
int umma_f8_gemm(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n, uint64_t k,
                 cudaStream_t st);
// The same tile over MXFP4 weights (block-scaled MMA with the weights' own E8M0 scales): fp32
// activations, 2..21 rows; or E4M3 activation codes with per-row factors (W4A8), up to 64 rows.
int umma_mxfp4_gemm(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k, cudaStream_t st);
int umma_mxfp4_w4a8(const void* a8, const float* as, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    cudaStream_t st);
int umma_f8_wait_timeouts(unsigned int* count);
int umma_f8_set_error_word(unsigned int* word);
// ---- merged small steps of a token (forward_elementwise.cu, attention.cu): what the deferred queue issues
// when it finds these steps side by side; each merged kernel repeats the single steps' arithmetic.
// Linear-attention layer: ssm_gate, conv1d_state (one row, no history slots), l2norm of the q and k heads in
// place, repeat_heads of both: a CTA per head-sized slice of the convolution's channels.
struct LinearMixerInputs {
  const float *a_log, *dt, *alpha_raw, *beta_raw;
  float *alpha, *beta;
  int gate_heads;
  const float *qkv, *conv_w;
  float *hist, *q, *k, *v;
  int conv_dim, width, key_dim;
  size_t qkv_offset;
  float *q_exp, *k_exp;
  int k_heads, cols, factor;
  float eps_q, scale_q, eps_k, scale_k;
};
int launch_linear_mixer_inputs(const LinearMixerInputs& p, cudaStream_t st);
// Full-attention layer: rmsnorm of the q and k heads in place, mrope of both (one row), and the append of the
// token's k and v rows to an fp32 cache (k_row / v_row null: no append).
struct HeadNormRope {
  float *q, *k;
  const float *q_w, *k_w;
  const unsigned long long* pos;
  int heads, kv_heads, head_dim, rope_dim, sec_t, sec_h;
  float eps_q, eps_k, theta;
  float* k_row;
  const float* v_src;
  float* v_row;
};
int launch_head_norm_rope(const HeadNormRope& p, cudaStream_t st);
// tsr_attention with out = attention * sigmoid(gate) written by the merge kernel (gate null: plain).
int attention_gated(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                    float* out, const float* gate, uint64_t m, uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim,
                    uint64_t q_base, uint64_t row_base, uint64_t window, uint64_t causal, cudaStream_t st);
// Point the kernels of each file at the host-visible error word (see pipeline.cuh); once per device.
int staged_set_error_word(unsigned int* word);
int staged_q6k_set_error_word(unsigned int* word);
int staged_f16_set_error_word(unsigned int* word);
int umma_set_error_word(unsigned int* word);

}  // namespace tsr
