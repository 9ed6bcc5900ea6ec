// Tensor-parallel sum all-reduce over NVLink peer memory: the stand-alone
// kernel and the communicator behind the C ABI's tsr_tp_* calls.  The protocol
// and the layout of the exchange memory are described in tp_device.cuh; the
// row-parallel GEMV kernels run the same device code as their last step.
//
// Exchange memory comes from cudaMalloc and is shared with peers through
// cudaIpc handles or, inside one process, peer access.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "context.h"
#include "launch.h"
#include "tessera_b200.h"
#include "tp_device.cuh"

namespace {

using namespace tsr;

constexpr int kChunkFloats = 1024;  // elements per CTA: 256 threads x 4

// Sum over ranks of `count` floats: thread t of CTA b owns elements 4 * (256 b + t) .. + 3.
// `src` holds `split` regions of `count` floats that are added in region order first
// (exactly as gemm_vec_reduce adds them, starting from 0.0f).
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(const float* src, int split, float* dst, size_t count, const TpTail tp) {
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) s_epoch = tp_call_epoch(tp);
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const size_t gtid = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  tp_reset_previous(tp, epoch, gtid, static_cast<size_t>(gridDim.x) * 256);
  const size_t e0 = gtid * 4;
  if (e0 < count) {
    float mine[4] = {0.f, 0.f, 0.f, 0.f};
    const int lanes = count - e0 < 4 ? static_cast<int>(count - e0) : 4;
    for (int s = 0; s < split; ++s)
      for (int j = 0; j < lanes; ++j) {
        const float v = src[static_cast<size_t>(s) * count + e0 + j];
        mine[j] = split == 1 ? v : mine[j] + v;
      }
    const size_t off = tp_slot_offset(tp, epoch, tp.rank) + e0;
    for (int j = 0; j < lanes; ++j) tp_push(tp, off + j, mine[j]);
    for (int j = 0; j < lanes; ++j) dst[e0 + j] = tp_wait_sum(tp, epoch, e0 + j);
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_cta_leaves(tp, epoch, gridDim.x, static_cast<unsigned int>(count));
}

}  // namespace

struct tsr_tp_comm {
  int device = 0, rank = 0, world = 1;
  size_t capacity = 0;  // floats per slot
  unsigned char* block = nullptr;  // local exchange memory
  size_t block_bytes = 0;
  void* peer_block[kMaxWorld] = {};
  bool peer_is_ipc[kMaxWorld] = {};
  bool attached[kMaxWorld] = {};

  static constexpr size_t kPrefixBytes = (kTpHeaderWords + kTpStateWords) * 4;
  size_t slots_bytes() const { return 3ull * world * capacity * 4; }
  unsigned int* state(void* base) const { return reinterpret_cast<unsigned int*>(base) + kTpHeaderWords; }
  float* slots(void* base) const { return reinterpret_cast<float*>(static_cast<unsigned char*>(base) + kPrefixBytes); }
  // Every rank computes its peers' offsets from its own capacity and world, so a
  // peer created with other values must be refused: its header says what it holds.
  int check_peer_header(const void* peer) const {
    unsigned int h[4] = {};
    if (cudaMemcpy(h, peer, sizeof(h), cudaMemcpyDefault) != cudaSuccess) {
      cudaGetLastError();
      return tsr::kDeviceError;
    }
    if (h[0] != kTpMagic || h[1] != static_cast<unsigned int>(world) || h[2] != static_cast<unsigned int>(capacity))
      return tsr::kInvalidArgument;
    return tsr::kOk;
  }
  bool tail(TpTail* out) const {
    out->world = world;
    out->rank = rank;
    out->capacity = capacity;
    for (int p = 0; p < world; ++p) {
      if (!attached[p]) return false;
      out->slots[p] = slots(peer_block[p]);
    }
    out->state = state(block);
    return true;
  }
};

namespace tsr {
// The tail parameters of a bound communicator, for the row-parallel GEMV launches.
int tp_tail_of(const tsr_tp_comm* comm, TpTail* out) {
  if (!comm || !out) return kInvalidArgument;
  return comm->tail(out) ? kOk : kInvalidArgument;
}
int tp_device_of(const tsr_tp_comm* comm) { return comm ? comm->device : -1; }
}  // namespace tsr

namespace {
int launch_allreduce(tsr_tp_comm* c, const float* src, uint64_t split, float* data, uint64_t count, void* stream) {
  if (!c || !src || !data || count == 0 || count > c->capacity || split == 0 || split > 65535 ||
      (reinterpret_cast<uintptr_t>(data) & 3u) || (reinterpret_cast<uintptr_t>(src) & 3u))
    return tsr::kInvalidArgument;
  // The current device is per host thread; one thread may drive several ranks.
  if (cudaSetDevice(c->device) != cudaSuccess) return tsr::kDeviceError;
  TpTail tail{};
  if (!c->tail(&tail)) return tsr::kInvalidArgument;
  const unsigned grid = static_cast<unsigned>((count + kChunkFloats - 1) / kChunkFloats);
  tp_allreduce_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, static_cast<int>(split), data, count,
                                                                          tail);
  return tsr::check_launch();
}
}  // namespace

namespace tsr {
int tp_allreduce_matrix(tsr_tp_comm* comm, float* data, uint64_t m, uint64_t n, cudaStream_t st) {
  return launch_allreduce(comm, data, 1, data, m * n, st);
}
}  // namespace tsr

extern "C" {

int tsr_tp_create(int device, int rank, int world, uint64_t max_floats, tsr_tp_comm** out) {
  if (!out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_floats == 0)
    return tsr::kInvalidArgument;
  if (cudaSetDevice(device) != cudaSuccess) return tsr::kDeviceError;
  auto* c = new tsr_tp_comm();
  c->device = device;
  c->rank = rank;
  c->world = world;
  c->capacity = (max_floats + kChunkFloats - 1) / kChunkFloats * kChunkFloats;
  if (c->capacity > 0xFFFFFFFFull) {
    delete c;
    return tsr::kInvalidArgument;
  }
  c->block_bytes = tsr_tp_comm::kPrefixBytes + c->slots_bytes();
  if (cudaMalloc(&c->block, c->block_bytes) != cudaSuccess) {
    cudaGetLastError();
    delete c;
    return tsr::kOutOfMemory;
  }
  cudaMemset(c->block, 0, tsr_tp_comm::kPrefixBytes);
  cudaMemset(c->block + tsr_tp_comm::kPrefixBytes, 0xFF, c->slots_bytes());  // every slot word: "not arrived"
  const unsigned int header[4] = {kTpMagic, static_cast<unsigned int>(world), static_cast<unsigned int>(c->capacity), 0u};
  cudaMemcpy(c->block, header, sizeof(header), cudaMemcpyHostToDevice);
  cudaDeviceSynchronize();
  c->peer_block[rank] = c->block;
  c->attached[rank] = true;
  *out = c;
  return tsr::kOk;
}

void tsr_tp_destroy(tsr_tp_comm* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (p != c->rank && c->attached[p] && c->peer_is_ipc[p]) cudaIpcCloseMemHandle(c->peer_block[p]);
  cudaFree(c->block);
  delete c;
}

int tsr_tp_local_block(tsr_tp_comm* c, void** ptr, uint64_t* bytes) {
  if (!c || !ptr) return tsr::kInvalidArgument;
  *ptr = c->block;
  if (bytes) *bytes = c->block_bytes;
  return tsr::kOk;
}

int tsr_tp_ipc_handle(tsr_tp_comm* c, void* handle64) {
  if (!c || !handle64) return tsr::kInvalidArgument;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, c->block) != cudaSuccess) return tsr::kDeviceError;
  std::memcpy(handle64, &h, 64);
  return tsr::kOk;
}

int tsr_tp_attach_ipc(tsr_tp_comm* c, int peer_rank, const void* handle64) {
  if (!c || !handle64 || peer_rank < 0 || peer_rank >= c->world || peer_rank == c->rank)
    return tsr::kInvalidArgument;
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* ptr = nullptr;
  if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return tsr::kDeviceError;
  }
  if (int rc = c->check_peer_header(ptr)) {
    cudaIpcCloseMemHandle(ptr);
    return rc;
  }
  c->peer_block[peer_rank] = ptr;
  c->peer_is_ipc[peer_rank] = true;
  c->attached[peer_rank] = true;
  return tsr::kOk;
}

int tsr_tp_attach_local(tsr_tp_comm* c, int peer_rank, int peer_device, void* peer_block) {
  if (!c || !peer_block || peer_rank < 0 || peer_rank >= c->world || peer_rank == c->rank)
    return tsr::kInvalidArgument;
  cudaSetDevice(c->device);
  if (peer_device != c->device) {
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, c->device, peer_device) != cudaSuccess || !can)
      return tsr::kUnsupportedFeature;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return tsr::kDeviceError;
    cudaGetLastError();
  }
  if (int rc = c->check_peer_header(peer_block)) return rc;
  c->peer_block[peer_rank] = peer_block;
  c->attached[peer_rank] = true;
  return tsr::kOk;
}

int tsr_tp_allreduce(tsr_tp_comm* c, float* data, uint64_t count, void* stream) {
  return launch_allreduce(c, data, 1, data, count, stream);
}

int tsr_tp_reduce_allreduce(tsr_tp_comm* c, const float* partials, uint64_t split, float* out, uint64_t count,
                            void* stream) {
  return launch_allreduce(c, partials, split, out, count, stream);
}

int tsr_tp_error_count(tsr_tp_comm* c, uint32_t* count) {
  if (!c || !count) return tsr::kInvalidArgument;
  cudaSetDevice(c->device);
  return cudaMemcpy(count, c->state(c->block) + 2, 4, cudaMemcpyDeviceToHost) == cudaSuccess ? tsr::kOk
                                                                                              : tsr::kDeviceError;
}

}  // extern "C"
