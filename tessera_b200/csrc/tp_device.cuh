// Device side of the tensor-parallel sum over ranks, shared by the stand-alone
// all-reduce kernel (tp.cu) and by the row-parallel GEMV kernels that finish
// with it (gemv_mma.cu, gemv_q6k_mma.cu).
//
// The reference sums the row-parallel partials by a rank-0 gather/add/broadcast
// between host barriers (src/models/qwen3_5/trunk.cpp:226-266 of the
// reference).  Here the unit of exchange is a "tile": a set of output elements
// that one CTA owns.  The CTA stores its partial values into slot `rank` of
// every rank's exchange memory (plain peer stores), publishes the tile's flag
// on every rank with a system-scope release, waits (bounded) until all ranks'
// flags of that tile have reached the call's epoch, and adds the slots in rank
// order 0, 1, 2, ... so that every rank ends with the same bits, equal to the
// reference's rank-0 accumulation order.
//
// Exchange memory of one rank:
//   header  [16] u32    magic, world, capacity, tiles_cap (checked on attach)
//   state   [16] u32    [0] calls completed, [1] CTAs that left the running call, [2] waits given up
//   slots   [parity 2][source rank W][capacity] fp32
//   flags   [source rank W][tiles_cap] u32   epoch of the last push of that tile
// All tiles of one call use the same epoch = calls completed + 1, read from
// device memory when the kernel starts and stored back by the last CTA to
// leave, so a captured CUDA graph can replay the collective.  Slots are double
// buffered by the epoch's parity: a rank cannot finish call e + 1 before every
// peer has entered it, hence has finished reading call e.
//
// Only ld/st.global on peer memory: no TMA, no multicast.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace tsr {

constexpr unsigned int kTpWaitPolls = 1u << 22;  // about a second of polling with back-off
constexpr unsigned int kTpMagic = 0x54505352u;
constexpr int kTpHeaderWords = 16, kTpStateWords = 16;

__device__ __forceinline__ unsigned int tp_ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Epoch of the call this kernel belongs to.  Read it after the kernel's
// dependency on the previous kernel of the stream is resolved.
__device__ __forceinline__ unsigned int tp_call_epoch(const TpTail& tp) {
  return *reinterpret_cast<volatile const unsigned int*>(tp.state) + 1u;
}

// Offset of (parity of `epoch`, source rank r) in a rank's slot memory.
__device__ __forceinline__ size_t tp_slot_offset(const TpTail& tp, unsigned int epoch, int r) {
  return (static_cast<size_t>(epoch & 1u) * tp.world + r) * tp.capacity;
}

// After this CTA's stores into the peers' slots: publish tile `tile` on every
// rank and wait for every rank's flag of that tile.  Called by all `nthreads`
// threads of the group that synchronises on named barrier `bar_id` (0 with the
// whole CTA); `tid` is the thread's index in that group (nthreads >= world).
__device__ __forceinline__ void tp_publish_and_wait(const TpTail& tp, unsigned int epoch, int tile, int tid,
                                                    int bar_id, int nthreads) {
  __threadfence_system();
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
  if (tid < tp.world) {
    tp_st_release_sys(tp.flags[tid] + static_cast<size_t>(tp.rank) * tp.tiles_cap + tile, epoch);
    const unsigned int* f = tp.flags[tp.rank] + static_cast<size_t>(tid) * tp.tiles_cap + tile;
    unsigned int polls = 0;
    // epochs grow monotonically; a later epoch cannot appear before this one is consumed
    while (static_cast<int>(tp_ld_acquire_sys(f) - epoch) < 0) {
      if (++polls > kTpWaitPolls) {
        atomicAdd(tp.state + 2, 1u);
        break;
      }
      if (polls > 64) __nanosleep(100);
    }
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
}

// Sum over ranks, in rank order, of element `e` of this rank's slots.
__device__ __forceinline__ float tp_rank_order_sum(const TpTail& tp, unsigned int epoch, size_t e) {
  const float* base = tp.slots[tp.rank] + tp_slot_offset(tp, epoch, 0) + e;
  float acc = __ldcg(base);
  for (int r = 1; r < tp.world; ++r) acc += __ldcg(base + static_cast<size_t>(r) * tp.capacity);
  return acc;
}

// One thread of every CTA calls this when the CTA has finished all its tiles:
// the last CTA of the grid to arrive completes the call.
__device__ __forceinline__ void tp_cta_leaves(const TpTail& tp, unsigned int epoch, unsigned int ctas) {
  __threadfence();
  const unsigned int t = atomicAdd(tp.state + 1, 1u);
  if (t == ctas - 1) {
    tp.state[1] = 0u;
    __threadfence();
    *reinterpret_cast<volatile unsigned int*>(tp.state) = epoch;
  }
}

}  // namespace tsr
