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

constexpr int kChunkFloats = 1024;  // tile of the flat all-reduce: 256 threads x float4

// Sum over ranks of an [m][n] matrix (n a multiple of 4), one CTA per tile of
// `tile_rows` columns of it (tile_rows a multiple of 4): tile t holds elements
// i*n + t*tile_rows + r for all i < m, r < tile_rows.  The flat all-reduce of
// `count` floats is the case m = 1, n = count, tile_rows = 1024.  `src` holds
// `split` regions of m*n floats that are added in region order first.
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(const float* src, int split, float* dst, int m, size_t n, int tile_rows, const TpTail tp) {
  __shared__ unsigned int s_epoch;
  const int tile = blockIdx.x;
  if (threadIdx.x == 0) s_epoch = tp_call_epoch(tp);
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int row_quads = tile_rows >> 2, quads = m * row_quads;
  const size_t region = static_cast<size_t>(m) * n;
  const size_t mine_off = tp_slot_offset(tp, epoch, tp.rank);
  for (int q = threadIdx.x; q < quads; q += 256) {
    const int i = q / row_quads, rq = q - i * row_quads;
    const size_t row = static_cast<size_t>(tile) * tile_rows + rq * 4;
    if (row >= n) continue;
    const size_t e = static_cast<size_t>(i) * n + row;
    float4 mine;
    if (split == 1) {
      mine = *reinterpret_cast<const float4*>(src + e);
    } else {
      // the split-K partial regions of a row-parallel projection, added in region
      // order exactly as gemm_vec_reduce adds them (starting from 0.0f)
      mine = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < split; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + static_cast<size_t>(s) * region + e);
        mine.x += v.x;
        mine.y += v.y;
        mine.z += v.z;
        mine.w += v.w;
      }
    }
    // push: my partial into slot `rank` of every rank (my own included)
    for (int r = 0; r < tp.world; ++r) *reinterpret_cast<float4*>(tp.slots[r] + mine_off + e) = mine;
  }
  tp_publish_and_wait(tp, epoch, tile, threadIdx.x, 0, 256);
  const float* base = tp.slots[tp.rank] + tp_slot_offset(tp, epoch, 0);
  for (int q = threadIdx.x; q < quads; q += 256) {
    const int i = q / row_quads, rq = q - i * row_quads;
    const size_t row = static_cast<size_t>(tile) * tile_rows + rq * 4;
    if (row >= n) continue;
    const size_t e = static_cast<size_t>(i) * n + row;
    float4 acc = __ldcg(reinterpret_cast<const float4*>(base + e));
    for (int r = 1; r < tp.world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(base + static_cast<size_t>(r) * tp.capacity + e));
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4*>(dst + e) = acc;
  }
  if (threadIdx.x == 0) tp_cta_leaves(tp, epoch, gridDim.x);
}

}  // namespace

struct tsr_tp_comm {
  int device = 0, rank = 0, world = 1;
  size_t capacity = 0;  // floats per slot
  unsigned int tiles_cap = 0;
  unsigned char* block = nullptr;  // local exchange memory
  size_t block_bytes = 0;
  void* peer_block[kMaxWorld] = {};
  bool peer_is_ipc[kMaxWorld] = {};
  bool attached[kMaxWorld] = {};

  static constexpr size_t kPrefixBytes = (kTpHeaderWords + kTpStateWords) * 4;
  size_t slots_bytes() const { return 2ull * world * capacity * 4; }
  unsigned int* state(void* base) const { return reinterpret_cast<unsigned int*>(base) + kTpHeaderWords; }
  float* slots(void* base) const { return reinterpret_cast<float*>(static_cast<unsigned char*>(base) + kPrefixBytes); }
  unsigned int* flags(void* base) const {
    return reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(base) + kPrefixBytes + slots_bytes());
  }
  // Every rank computes its peers' offsets from its own capacity and world, so a
  // peer created with other values must be refused: its header says what it holds.
  int check_peer_header(const void* peer) const {
    unsigned int h[4] = {};
    if (cudaMemcpy(h, peer, sizeof(h), cudaMemcpyDefault) != cudaSuccess) {
      cudaGetLastError();
      return tsr::kDeviceError;
    }
    if (h[0] != kTpMagic || h[1] != static_cast<unsigned int>(world) || h[2] != static_cast<unsigned int>(capacity) ||
        h[3] != tiles_cap)
      return tsr::kInvalidArgument;
    return tsr::kOk;
  }
  bool tail(TpTail* out) const {
    out->world = world;
    out->rank = rank;
    out->tiles_cap = tiles_cap;
    out->capacity = capacity;
    for (int p = 0; p < world; ++p) {
      if (!attached[p]) return false;
      out->slots[p] = slots(peer_block[p]);
      out->flags[p] = flags(peer_block[p]);
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
int launch_tiled(tsr_tp_comm* c, const float* src, uint64_t split, float* data, uint64_t m, uint64_t n,
                 uint64_t tile_rows, cudaStream_t stream) {
  if (!c || !src || !data || m == 0 || n == 0 || m > 65535 || m * n > c->capacity || n % 4 != 0 || tile_rows == 0 ||
      tile_rows % 4 != 0 || split == 0 || split > 65535 || (reinterpret_cast<uintptr_t>(data) & 15u) ||
      (reinterpret_cast<uintptr_t>(src) & 15u))
    return tsr::kInvalidArgument;
  const uint64_t tiles = (n + tile_rows - 1) / tile_rows;
  if (tiles > c->tiles_cap) return tsr::kInvalidArgument;
  // The current device is per host thread; one thread may drive several ranks.
  if (cudaSetDevice(c->device) != cudaSuccess) return tsr::kDeviceError;
  TpTail tail{};
  if (!c->tail(&tail)) return tsr::kInvalidArgument;
  tp_allreduce_kernel<<<static_cast<unsigned>(tiles), 256, 0, stream>>>(src, static_cast<int>(split), data,
                                                                        static_cast<int>(m), n,
                                                                        static_cast<int>(tile_rows), tail);
  return tsr::check_launch();
}
int launch_allreduce(tsr_tp_comm* c, const float* src, uint64_t split, float* data, uint64_t count, void* stream) {
  return launch_tiled(c, src, split, data, 1, count, kChunkFloats, static_cast<cudaStream_t>(stream));
}
}  // namespace

namespace tsr {
int tp_allreduce_tiled(tsr_tp_comm* comm, float* data, uint64_t m, uint64_t n, uint64_t tile_rows, cudaStream_t st) {
  return launch_tiled(comm, data, 1, data, m, n, tile_rows, st);
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
  c->tiles_cap = static_cast<unsigned int>(c->capacity / 16);  // a GEMV tile has at least 16 outputs
  c->block_bytes = tsr_tp_comm::kPrefixBytes + c->slots_bytes() + static_cast<size_t>(world) * c->tiles_cap * 4;
  if (cudaMalloc(&c->block, c->block_bytes) != cudaSuccess) {
    cudaGetLastError();
    delete c;
    return tsr::kOutOfMemory;
  }
  cudaMemset(c->block, 0, c->block_bytes);
  const unsigned int header[4] = {kTpMagic, static_cast<unsigned int>(world), static_cast<unsigned int>(c->capacity),
                                  c->tiles_cap};
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
