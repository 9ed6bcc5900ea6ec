// Tensor-parallel sum all-reduce over NVLink peer memory.
//
// The reference reduces the row-parallel partials by a rank-0
// gather/add/broadcast between host barriers
// (src/models/qwen3_5/trunk.cpp:226-266 of the reference).  Here every rank
// pushes its partial straight into a slot of every peer's exchange buffer
// with plain peer stores, publishes a per-chunk epoch flag with a
// system-scope release, waits (bounded) for the other ranks' flags and adds
// the slots in rank order 0,1,2..., so every rank ends with bit-identical
// sums and the result equals the reference's rank-0 accumulation order.
//
// Exchange memory of one rank (cudaMalloc, shared with peers through
// cudaIpc handles or, inside one process, peer access):
//   slots [parity 2][source rank W][capacity] fp32
//   flags [source rank W][chunks]            u32  epoch of the last push
//   count [chunks]                           u32  this rank's own epoch
//   error                                    u32  bounded waits that gave up
// The epoch of a chunk lives in device memory and is advanced by the kernel,
// so a captured CUDA graph can replay the collective.  Slots are double
// buffered by epoch parity: a rank can be at most one call ahead of a peer.
//
// No TMA and no multicast are used on peer memory: only ld/st.global.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "launch.h"
#include "tessera_b200.h"

namespace {

constexpr int kMaxWorld = 8;
constexpr int kChunkFloats = 1024;  // one CTA of 256 threads x float4
constexpr unsigned int kWaitPolls = 1u << 22;  // ~ a second of polling with backoff

struct Peers {
  float* slots[kMaxWorld];
  unsigned int* flags[kMaxWorld];
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256)
tp_allreduce_kernel(const float* src, int split, float* dst, size_t count, Peers peers, int rank, int world,
                    size_t capacity, int chunks_cap, unsigned int* my_count, unsigned int* error) {
  __shared__ unsigned int s_epoch;
  const int chunk = blockIdx.x;
  if (threadIdx.x == 0) s_epoch = my_count[chunk] + 1;
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const size_t parity_off = static_cast<size_t>(epoch & 1u) * world * capacity;
  const size_t idx = static_cast<size_t>(chunk) * kChunkFloats + threadIdx.x * 4;
  const bool active = idx < count;
  float4 mine = make_float4(0.f, 0.f, 0.f, 0.f);
  if (active) {
    if (split == 1) {
      mine = *reinterpret_cast<const float4*>(src + idx);
    } else {
      // the split-K partial regions of a row-parallel projection, added in region
      // order exactly as gemm_vec_reduce adds them (starting from 0.0f)
      for (int s = 0; s < split; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + static_cast<size_t>(s) * count + idx);
        mine.x += v.x;
        mine.y += v.y;
        mine.z += v.z;
        mine.w += v.w;
      }
    }
    // push: my partial into slot `rank` of every rank (my own included)
    for (int p = 0; p < world; ++p) {
      float* dst = peers.slots[p] + parity_off + static_cast<size_t>(rank) * capacity + idx;
      *reinterpret_cast<float4*>(dst) = mine;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world)
    st_release_sys(peers.flags[threadIdx.x] + static_cast<size_t>(rank) * chunks_cap + chunk, epoch);
  // wait for every source rank's flag of this chunk
  if (threadIdx.x < world) {
    const unsigned int* f = peers.flags[rank] + static_cast<size_t>(threadIdx.x) * chunks_cap + chunk;
    unsigned int polls = 0;
    // epochs grow monotonically; a later epoch cannot appear before this one is consumed
    while (static_cast<int>(ld_acquire_sys(f) - epoch) < 0) {
      if (++polls > kWaitPolls) {
        atomicAdd(error, 1u);
        break;
      }
      if (polls > 64) __nanosleep(200);
    }
  }
  __syncthreads();
  if (active) {
    const float* base = peers.slots[rank] + parity_off + idx;
    float4 acc = *reinterpret_cast<const float4*>(base);
    for (int r = 1; r < world; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(base + static_cast<size_t>(r) * capacity);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4*>(dst + idx) = acc;
  }
  if (threadIdx.x == 0) my_count[chunk] = epoch;
}

}  // namespace

struct tsr_tp_comm {
  int device = 0, rank = 0, world = 1;
  size_t capacity = 0;  // floats per slot
  int chunks = 0;
  unsigned char* block = nullptr;  // local exchange memory
  size_t block_bytes = 0;
  void* peer_block[kMaxWorld] = {};
  bool peer_is_ipc[kMaxWorld] = {};
  bool attached[kMaxWorld] = {};

  size_t slots_bytes() const { return 2ull * world * capacity * 4; }
  float* slots(void* base) const { return reinterpret_cast<float*>(base); }
  unsigned int* flags(void* base) const {
    return reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(base) + slots_bytes());
  }
  unsigned int* counts() const { return flags(block) + static_cast<size_t>(world) * chunks; }
  unsigned int* error() const { return counts() + chunks; }
};

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
  c->chunks = static_cast<int>(c->capacity / kChunkFloats);
  c->block_bytes = c->slots_bytes() + (static_cast<size_t>(world) * c->chunks + c->chunks + 64) * 4;
  if (cudaMalloc(&c->block, c->block_bytes) != cudaSuccess) {
    delete c;
    return tsr::kOutOfMemory;
  }
  cudaMemset(c->block, 0, c->block_bytes);
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
  c->peer_block[peer_rank] = peer_block;
  c->attached[peer_rank] = true;
  return tsr::kOk;
}

namespace {
int launch_allreduce(tsr_tp_comm* c, const float* src, uint64_t split, float* dst, uint64_t count, void* stream);
}

int tsr_tp_allreduce(tsr_tp_comm* c, float* data, uint64_t count, void* stream) {
  return launch_allreduce(c, data, 1, data, count, stream);
}

int tsr_tp_reduce_allreduce(tsr_tp_comm* c, const float* partials, uint64_t split, float* out, uint64_t count,
                            void* stream) {
  return launch_allreduce(c, partials, split, out, count, stream);
}

namespace {
int launch_allreduce(tsr_tp_comm* c, const float* src, uint64_t split, float* data, uint64_t count, void* stream) {
  if (!c || !src || !data || count == 0 || count > c->capacity || count % 4 != 0 || split == 0 || split > 65535 ||
      (reinterpret_cast<uintptr_t>(data) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u))
    return tsr::kInvalidArgument;
  // The current device is per host thread; one thread may drive several ranks.
  if (cudaSetDevice(c->device) != cudaSuccess) return tsr::kDeviceError;
  Peers peers{};
  for (int p = 0; p < c->world; ++p) {
    if (!c->attached[p]) return tsr::kInvalidArgument;
    peers.slots[p] = c->slots(c->peer_block[p]);
    peers.flags[p] = c->flags(c->peer_block[p]);
  }
  const unsigned grid = static_cast<unsigned>((count + kChunkFloats - 1) / kChunkFloats);
  tp_allreduce_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<int>(split), data, count, peers, c->rank, c->world, c->capacity, c->chunks, c->counts(),
      c->error());
  return tsr::check_launch();
}
}  // namespace

int tsr_tp_error_count(tsr_tp_comm* c, uint32_t* count) {
  if (!c || !count) return tsr::kInvalidArgument;
  cudaSetDevice(c->device);
  return cudaMemcpy(count, c->error(), 4, cudaMemcpyDeviceToHost) == cudaSuccess ? tsr::kOk
                                                                                  : tsr::kDeviceError;
}

}  // extern "C"
