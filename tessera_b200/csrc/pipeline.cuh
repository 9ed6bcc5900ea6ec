// mbarrier / TMA / mma.sync primitives shared by the staged GEMV kernels
// (sm_100a inline PTX).  Every wait is bounded: after kSpinLimit polls the
// waiter adds one to the counter it was given (a file-scope __device__ word of
// the including translation unit, read back by the host after
// synchronisation) and the caller leaves its loop, so a lost copy can never
// hang the device.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tsr {

constexpr uint32_t kSpinLimit = 1u << 22;  // each poll may itself suspend for a while: seconds at most

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---- thread-block clusters: a barrier over all threads of the cluster, a peer CTA's
// shared memory (distributed shared memory), and an mbarrier signalled across CTAs
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Arrives (release, cluster scope) on an mbarrier in a peer CTA's shared memory.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{.reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Host-visible error word (pinned, mapped memory shared by every kernel file of the
// library): a wait that gives up also raises it, so the host learns of a failure by
// reading one word of its own memory instead of copying counters back from the device.
// Each translation unit holds its own copy of the pointer, set per device by
// set_host_error_word() of that unit.
static __device__ unsigned int* g_host_error_word = nullptr;
static inline int set_host_error_word(unsigned int* word) {
  return cudaMemcpyToSymbol(g_host_error_word, &word, sizeof(word)) == cudaSuccess ? 0 : 6;
}

// Returns false when the wait gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* timeouts) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbar_try_wait(bar, parity)) return true;
  atomicAdd(timeouts, 1u);
  if (g_host_error_word != nullptr) *reinterpret_cast<volatile unsigned int*>(g_host_error_word) = 1u;
  return false;
}

// The same with an acquire at cluster scope: what peer CTAs stored before their arrival
// (mbar_arrive_remote) is visible after it.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, unsigned int* timeouts) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  atomicAdd(timeouts, 1u);
  if (g_host_error_word != nullptr) *reinterpret_cast<volatile unsigned int*>(g_host_error_word) = 1u;
  return false;
}

// Ring slot and use count of chunk c when `groups` consumer groups (two unless
// said otherwise) take the chunks round-robin.  Each group owns its own slots
// (group g the slots g, g + groups, ...; the ring has at least one per group),
// so every slot is waited on by one group, in order.  A parity wait only tells the phase
// before from the phase after: if a slot alternated between the groups, a
// group that runs ahead would wait on a phase the barrier has not reached and
// the wait would return at once.
struct RingUse {
  int slot, round;
};
__device__ __forceinline__ RingUse ring_use(int c, int stages, int groups = 2) {
  const int group = c % groups, j = c / groups;
  const int owned = (stages - group + groups - 1) / groups;
  const int idx = j % owned;
  return {group + groups * idx, j / owned};
}

// The producer's walk through the chunks that follow the first `stages` ones (which fill the
// ring slot by slot): the same (slot, round) sequence as ring_use(j) for j = stages, stages + 1,
// ..., kept in registers without divisions -- the producer thread sits on the refill path of
// every stage, and each instruction between a consumer's release and the next copy counts.
template <int GROUPS>
struct RingCursor {
  int idx[GROUPS], rnd[GROUPS], owned[GROUPS];
  int grp;
  __device__ __forceinline__ void start_after_fill(int stages) {
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      owned[g] = (stages - g + GROUPS - 1) / GROUPS;
      idx[g] = 0;  // every group has used each of its slots once
      rnd[g] = 1;
    }
    grp = stages % GROUPS;
  }
  __device__ __forceinline__ RingUse next() {
    RingUse use{0, 0};
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      if (grp == g) {
        use.slot = g + GROUPS * idx[g];
        use.round = rnd[g];
        if (++idx[g] == owned[g]) {
          idx[g] = 0;
          ++rnd[g];
        }
      }
    }
    grp = grp + 1 == GROUPS ? 0 : grp + 1;
    return use;
  }
};

// Tiled TMA load of one 3-D box into shared memory; completion is counted in
// bytes on `bar`.  The innermost coordinate must keep the 16-byte rule
// (c0 * element size a multiple of 16); every caller passes c0 = 0.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));  // (x & mask) | orv
  return r;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Host side: encode a tiled tensor map through the driver entry point
// (resolved at run time; the library does not link libcuda).
// swizzle128: shared-memory rows of 128 bytes with the 16-byte pieces of row r
// stored at piece index ^ (r mod 8) (CU_TENSOR_MAP_SWIZZLE_128B).
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      bool swizzle128 = false);

}  // namespace tsr
