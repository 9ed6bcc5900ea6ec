// The context behind the C ABI's tsr_context handle, shared by capi.cu (memory,
// copies, synchronisation) and dispatch.cu (the name-keyed launches and their
// deferred submission).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "launch.h"

struct tsr_tp_comm;

namespace tsr {

constexpr size_t kStageWindow = 4u << 20;  // bytes per pinned staging window
constexpr int kStageWindows = 8;
constexpr int kMaxLaunchBuffers = 16, kMaxLaunchScalars = 16;  // include/tessera/backend.hpp:47-48

// One name-keyed launch as the caller made it, kept until the queue is flushed.
struct PendingLaunch {
  int kernel;
  uint32_t grid_y;
  int nbuf, nsc;
  const void* buf[kMaxLaunchBuffers];
  size_t bytes[kMaxLaunchBuffers];
  uint64_t sc[kMaxLaunchScalars];
};

// A flushed queue that has been seen before, instantiated as a CUDA graph.
struct CachedGraph {
  cudaGraphExec_t exec = nullptr;
  uint64_t last_use = 0;
  uint64_t kernels = 0;  // kernel nodes it holds
  size_t ops = 0;        // launches of the queue it was captured from
};

struct LaunchStats {
  uint64_t api_launches = 0;     // tsr_launch calls accepted
  uint64_t device_kernels = 0;   // kernels those calls became (inside graphs too)
  uint64_t graph_launches = 0;   // cudaGraphLaunch calls
  uint64_t flushes = 0;          // non-empty queue flushes
};

}  // namespace tsr

struct tsr_context {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  std::string error;
  // Pinned staging ring for host<->device copies: a window is reused only
  // after the copy that read or wrote it has completed (event guard).
  unsigned char* stage = nullptr;
  cudaEvent_t stage_done[tsr::kStageWindows] = {};
  bool stage_busy[tsr::kStageWindows] = {};
  int stage_next = 0;
  bool peer_enabled[64] = {};
  unsigned int seen_error_word = 0, seen_timeouts = 0;
  std::mutex mutex;

  // Deferred submission (tsr_set_deferred): launches wait in `pending` until a
  // copy, a synchronisation or tsr_flush, are merged where the kernels allow
  // it, and a queue that repeats is replayed as a CUDA graph.
  bool deferred = false;
  bool use_graphs = true;
  bool fold_elementwise = true;  // silu_mul, rmsnorm and add may run inside the projection launches
  std::vector<tsr::PendingLaunch> pending;
  std::unordered_map<uint64_t, tsr::CachedGraph> graphs;
  std::unordered_map<uint64_t, int> seen_queues;  // hash -> times flushed without a graph
  uint64_t use_clock = 0;
  tsr::LaunchStats stats;
  // Scratch of the launches that split k among CTAs and add the chunks themselves.
  tsr::FusedScratch scratch = {};
  // Tensor-parallel communicator bound with tsr_tp_bind (not owned).
  tsr_tp_comm* tp = nullptr;

  int fail(cudaError_t e, const char* what);
  int select();
  unsigned char* window(int* index);
};

namespace tsr {
// Issues everything in ctx->pending on the context's stream (dispatch.cu).
int flush_pending(tsr_context* ctx);
// Device-to-device copies up to this size wait in the queue with the launches around them (dispatch.cu).
constexpr size_t kQueuedCopyLimit = 1u << 20;
int queue_copy(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t dst_offset, size_t bytes);
// The tail parameters / device of a communicator (tp.cu).
int tp_tail_of(const tsr_tp_comm* comm, TpTail* out);
int tp_device_of(const tsr_tp_comm* comm);
// Sum over ranks of an [m][n] fp32 matrix in place (tp.cu).
int tp_allreduce_matrix(tsr_tp_comm* comm, float* data, uint64_t m, uint64_t n, cudaStream_t st);
}  // namespace tsr
