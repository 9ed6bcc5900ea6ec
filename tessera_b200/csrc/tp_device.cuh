// Device side of the tensor-parallel sum over ranks, shared by the stand-alone
// all-reduce kernel (tp.cu) and by the row-parallel GEMV kernels that finish
// with it (gemv_mma.cu, gemv_q6k_mma.cu).
//
// The reference sums the row-parallel partials by a rank-0 gather/add/broadcast
// between host barriers (src/models/qwen3_5/trunk.cpp:226-266 of the
// reference).  Here every rank stores its partial values straight into slot
// `rank` of every rank's exchange memory (plain peer stores) and each rank adds
// the slots in rank order 0, 1, 2, ..., so every rank ends with the same bits,
// equal to the reference's rank-0 accumulation order.
//
// There are no flags and no fences: a slot word that has not arrived yet holds a
// sentinel bit pattern (a NaN payload that arithmetic never produces; a partial
// value that happens to carry it is sent as the canonical NaN), and the thread
// that needs element e polls the W slot words of e until none is the sentinel
// (bounded).  A 4-byte store is delivered whole, so a word is either the
// sentinel or the value.  The latency of the collective is one NVLink store
// plus the poll, instead of store + fence + flag + acquire.
//
// Exchange memory of one rank:
//   header  [16] u32    magic, world, capacity (checked on attach)
//   state   [16] u32    [0] calls completed, [1] CTAs that left the running call,
//                       [2] waits given up, [4..6] elements in use per buffer
//   slots   [buffer 3][source rank W][capacity] fp32, all sentinel at rest
// Call number c (= calls completed + 1, read from device memory when the kernel
// starts, stored back by the last CTA to leave, so a captured CUDA graph can
// replay the collective) uses buffer c % 3 and, while it runs, resets buffer
// (c - 1) % 3 to the sentinel over the extent the previous call used.  That
// buffer is next written by a peer in its call c + 2, which the peer cannot
// start before this rank's push of call c + 1 -- a kernel later, so the reset
// is complete and visible.  The buffer this rank reads now, c % 3, was reset
// during call c - 2... c - 1 at the latest, a kernel earlier than any peer's
// push of call c, for the same reason.
//
// Only ld/st.global on peer memory: no TMA, no multicast.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace tsr {

constexpr unsigned int kTpWaitPolls = 1u << 22;  // about a second of polling with back-off
constexpr unsigned int kTpMagic = 0x54505332u;
constexpr int kTpHeaderWords = 16, kTpStateWords = 16;
constexpr unsigned int kTpSentinel = 0xFFFFFFFFu;       // "not arrived"
constexpr unsigned int kTpCanonicalNan = 0x7FFFFFFFu;  // what a value with the sentinel's bits is sent as

// Kernel parameters are best read with constant indices (a run-time index into a
// parameter array makes the compiler copy the array to local memory or keep all of it in
// registers), so the per-rank pointers are picked by unrolled compares.
__device__ __forceinline__ float* tp_slots_of(const TpTail& tp, int r) {
  float* p = tp.slots[0];
#pragma unroll
  for (int i = 1; i < kMaxWorld; ++i)
    if (r == i) p = tp.slots[i];
  return p;
}

// Number of the call this kernel belongs to.  Read it after the kernel's
// dependency on the previous kernel of the stream is resolved.
__device__ __forceinline__ unsigned int tp_call_epoch(const TpTail& tp) {
  return *reinterpret_cast<volatile const unsigned int*>(tp.state) + 1u;
}

// Offset of (buffer of call `epoch`, source rank r) in a rank's slot memory.
__device__ __forceinline__ size_t tp_slot_offset(const TpTail& tp, unsigned int epoch, int r) {
  return (static_cast<size_t>(epoch % 3u) * tp.world + r) * tp.capacity;
}

__device__ __forceinline__ void tp_st(float* p, float v) {
  unsigned int bits = __float_as_uint(v);
  if (bits == kTpSentinel) bits = kTpCanonicalNan;
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(bits) : "memory");
}
__device__ __forceinline__ unsigned int tp_ld(const float* p) {
  unsigned int bits;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(bits) : "l"(p) : "memory");
  return bits;
}

// Stores v into element `off` of every rank's slot memory (this rank's own included).
__device__ __forceinline__ void tp_push(const TpTail& tp, size_t off, float v) {
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r)
    if (r < tp.world) tp_st(tp.slots[r] + off, v);
}

// Waits (bounded) for element e of every source rank in this rank's buffer of call
// `epoch` and returns their sum in rank order.  The W slot words are loaded together (one
// trip to memory when everything has arrived, not W trips one behind the other); only words
// that still hold the sentinel are polled again.
__device__ __forceinline__ float tp_wait_sum(const TpTail& tp, unsigned int epoch, size_t e) {
  const float* base = tp_slots_of(tp, tp.rank) + tp_slot_offset(tp, epoch, 0) + e;
  unsigned int bits[kMaxWorld];
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r)
    bits[r] = r < tp.world ? tp_ld(base + static_cast<size_t>(r) * tp.capacity) : 0u;
  for (unsigned int polls = 0;;) {
    bool missing = false;
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) missing = missing || bits[r] == kTpSentinel;
    if (!missing) break;
    if (++polls > kTpWaitPolls) {
      atomicAdd(tp.state + 2, 1u);
      break;
    }
    if (polls > 32) __nanosleep(40);
    // every word still missing is asked for again, all of them in flight together
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (bits[r] == kTpSentinel) bits[r] = tp_ld(base + static_cast<size_t>(r) * tp.capacity);
  }
  float acc = __uint_as_float(bits[0]);
#pragma unroll
  for (int r = 1; r < kMaxWorld; ++r)
    if (r < tp.world) acc += __uint_as_float(bits[r]);
  return acc;
}

// Every thread of the grid calls this once per call (anywhere after tp_call_epoch):
// thread `gtid` of `gthreads` resets its share of the previous call's buffer.
__device__ __forceinline__ void tp_reset_previous(const TpTail& tp, unsigned int epoch, size_t gtid, size_t gthreads) {
  const unsigned int prev = (epoch + 2u) % 3u;  // (epoch - 1) mod 3
  const size_t used = *reinterpret_cast<volatile const unsigned int*>(tp.state + 4 + prev);
  if (used == 0) return;
  float* base = tp_slots_of(tp, tp.rank) + static_cast<size_t>(prev) * tp.world * tp.capacity;
  const size_t quads = (used + 3) / 4;
  for (int r = 0; r < tp.world; ++r) {
    uint4* q = reinterpret_cast<uint4*>(base + static_cast<size_t>(r) * tp.capacity);
    for (size_t i = gtid; i < quads; i += gthreads) q[i] = make_uint4(kTpSentinel, kTpSentinel, kTpSentinel, kTpSentinel);
  }
}

// One thread of every CTA calls this when the CTA has finished all its work (reset
// included): the last CTA of the grid to arrive completes the call.  `used` = elements
// this call exchanged.
// The caller has synchronised the CTA's threads (a barrier) after their resets: the
// arrival's release then covers them, and the last CTA's acquire sees every CTA's resets
// before it marks the buffer clean.  The state words are read next by the following kernel
// of this stream, which the kernel boundary orders; no thread needs a full fence.
__device__ __forceinline__ void tp_cta_leaves(const TpTail& tp, unsigned int epoch, unsigned int ctas, unsigned int used) {
  unsigned int t;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(tp.state + 1) : "memory");
  if (t == ctas - 1) {
    tp.state[1] = 0u;
    tp.state[4 + epoch % 3u] = used;
    tp.state[4 + (epoch + 2u) % 3u] = 0u;  // the previous call's buffer is clean again
    *reinterpret_cast<volatile unsigned int*>(tp.state) = epoch;
  }
}

}  // namespace tsr
