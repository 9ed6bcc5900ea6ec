// Staged tensor-pipe GEMV for Q6_K weights (m = 1..8 activation rows).
//
// Same structure as the Q4_K kernel (gemv_mma.cu): one CTA per tile of 16..64 rows
// and split chunk, a TMA-fed ring of shared-memory stages, weights as the A
// operand of an int8 mma.sync, activations as signed base-256 digit columns,
// integer group scales applied to the s32 partial sums, the fp16 block scale
// in fp32.
//
// What Q6_K changes (block = ql[128] qh[64] int8 scales[16] fp16 d, 210 bytes;
// value = d * sc[g] * (q - 32), 16 elements per scale group;
// src/core/numerics/quant.cpp:421-449 of the reference):
//   * A row of 210-byte blocks is only 8-byte aligned (k/256 a multiple of 4),
//     and TMA wants 16-byte strides.  Two tensor maps solve it: one over the
//     even rows, one over the odd rows, each with a row pitch of two weight
//     rows (a multiple of 16 bytes) and, for the odd rows, a base moved down
//     to the 16-byte boundary.  A stage is the 464-byte window of each row
//     that contains two blocks, starting at the 16-byte boundary below them;
//     464 B = 80 mod 128 keeps the 4-byte fragment loads bank-conflict free.
//     A warp owns 16 consecutive rows: MMA rows 0..7 are its even rows, 8..15 its odd rows.
//   * Stages start at even block indices, so the first block of a stage is
//     word aligned and the second one sits 2 bytes off a word: its words are
//     assembled from two aligned loads with a funnel shift.
//   * One MMA (m16n8k16, u8 x s8) per 16-element scale group; the 6-bit value
//     is the nibble OR the two high bits moved into place.
//   * The "- 32" is one more pair of MMAs per block: the int8 scales against
//     the per-group activation digit sums, i.e. sum_g sc[g] * sum_k a[k].
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "codec.cuh"
#include "context.h"
#include "launch.h"
#include "pipeline.cuh"
#include "staged_common.cuh"
#include "tp_device.cuh"

namespace tsr {

__device__ unsigned int g_q6k_wait_timeouts = 0;

namespace {

using namespace staged;

// A CTA owns 16 * rgs rows of W (rgs = 1..4 row groups, chosen per launch):
// 8 * rgs even rows and 8 * rgs odd rows, one TMA box each per stage.
constexpr int kChunkBytes = 2 * kQ6KBlockBytes;          // 420: two blocks per stage
constexpr int kWindowWords = 58;                         // u64 per row window
constexpr int kRowPitch = kWindowWords * 8;              // 464 = 80 mod 128
constexpr int kGroupHalfBytes = 8 * kRowPitch;           // the even (or odd) rows of one row group: 3712
constexpr int kThreads = kStagedThreads;
constexpr int kGroups = 16;

__device__ __forceinline__ uint32_t lds32(const unsigned char* p) {
  return *reinterpret_cast<const uint32_t*>(p);
}
// 32-bit value at a shared-memory address that is 2 mod 4 (OFF2) or aligned.
template <bool OFF2>
__device__ __forceinline__ uint32_t ldw(const unsigned char* p) {
  if (OFF2) return __funnelshift_r(lds32(p - 2), lds32(p + 2), 16);
  return lds32(p);
}

// D(16x8, s32) = A(16x16, row) * B(16x8, s8, col), zero accumulate input
__device__ __forceinline__ void mma_k16_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void mma_k16_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// Sign-extended byte `idx` of a word of int8 scales: prmt copies the byte and
// replicates its sign into the three upper bytes (selector nibbles with bit 3 set).
__device__ __forceinline__ int sext_byte(uint32_t w, int idx) {
  const uint32_t sel = idx | ((8 | idx) << 4) | ((8 | idx) << 8) | ((8 | idx) << 12);
  int r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0), "r"(sel));
  return r;
}

struct ThreadCtx {
  const unsigned char* act_t;  // this thread's activation fragment base (column, 4*tig)
  const unsigned char* sum_t;  // this thread's digit-sum base (column, 4*tig)
  uint32_t act_sb, act_blk, sum_plane, sum_blk;
};

// One Q6_K block of one 16-row warp tile.  pa/pb: block start of the thread's two rows.
template <bool OFF2, int NCG>
__device__ __forceinline__ void q6k_block(const unsigned char* pa, const unsigned char* pb, int tig,
                                          int bl, const ThreadCtx (&tc)[NCG], const float* cs_t,
                                          float (&o)[NCG][4]) {
  constexpr uint32_t kNib = 0x0F0F0F0Fu, kTwo = 0x30303030u;
  uint32_t scA[4], scB[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    scA[i] = ldw<OFF2>(pa + 192 + 4 * i);
    scB[i] = ldw<OFF2>(pb + 192 + 4 * i);
  }
  int t1[NCG][4];
#pragma unroll
  for (int g = 0; g < NCG; ++g)
#pragma unroll
    for (int e = 0; e < 4; ++e) t1[g][e] = 0;

#pragma unroll
  for (int h = 0; h < 2; ++h) {      // 128-element half of the block
#pragma unroll
    for (int lh = 0; lh < 2; ++lh) {  // 16-element half of each 32-element run
      const int off = 16 * lh + 4 * tig;
      const uint32_t la0 = ldw<OFF2>(pa + 64 * h + off), la1 = ldw<OFF2>(pa + 64 * h + 32 + off);
      const uint32_t ha = ldw<OFF2>(pa + 128 + 32 * h + off);
      const uint32_t lb0 = ldw<OFF2>(pb + 64 * h + off), lb1 = ldw<OFF2>(pb + 64 * h + 32 + off);
      const uint32_t hb = ldw<OFF2>(pb + 128 + 32 * h + off);
      // 6-bit values of the four 32-element runs (low/high nibbles of ql, two bits of qh each)
      const uint32_t qa[4] = {(la0 & kNib) | ((ha << 4) & kTwo), (la1 & kNib) | ((ha << 2) & kTwo),
                              ((la0 >> 4) & kNib) | (ha & kTwo), ((la1 >> 4) & kNib) | ((ha >> 2) & kTwo)};
      const uint32_t qb[4] = {(lb0 & kNib) | ((hb << 4) & kTwo), (lb1 & kNib) | ((hb << 2) & kTwo),
                              ((lb0 >> 4) & kNib) | (hb & kTwo), ((lb1 >> 4) & kNib) | ((hb >> 2) & kTwo)};
#pragma unroll
      for (int pp = 0; pp < 4; ++pp) {
        // scale group 8h + 2pp + lh: byte 2(pp&1)+lh of scale word 2h + pp/2
        const int sa = sext_byte(scA[2 * h + (pp >> 1)], 2 * (pp & 1) + lh);
        const int sb = sext_byte(scB[2 * h + (pp >> 1)], 2 * (pp & 1) + lh);
#pragma unroll
        for (int g = 0; g < NCG; ++g) {
          const uint32_t f = lds32(tc[g].act_t + bl * tc[g].act_blk + (4 * h + pp) * tc[g].act_sb + 16 * lh);
          int pr[4];
          mma_k16_u8s8(pr, qa[pp], qb[pp], f);
          t1[g][0] += sa * pr[0];
          t1[g][1] += sa * pr[1];
          t1[g][2] += sb * pr[2];
          t1[g][3] += sb * pr[3];
        }
      }
    }
  }
  // the "- 32": sum over groups of sc[g] * (digit sum of the group); k slots = groups
  const float dA = fp16_bits_to_float(*reinterpret_cast<const unsigned short*>(pa + 208));
  const float dB = fp16_bits_to_float(*reinterpret_cast<const unsigned short*>(pb + 208));
  const uint32_t ma = tig == 0 ? scA[0] : tig == 1 ? scA[1] : tig == 2 ? scA[2] : scA[3];
  const uint32_t mb = tig == 0 ? scB[0] : tig == 1 ? scB[1] : tig == 2 ? scB[2] : scB[3];
#pragma unroll
  for (int g = 0; g < NCG; ++g) {
    const unsigned char* sp = tc[g].sum_t + bl * tc[g].sum_blk;
    int r0[4], r1[4];
    mma_k16_s8s8(r0, ma, mb, lds32(sp));
    mma_k16_s8s8(r1, ma, mb, lds32(sp + tc[g].sum_plane));
    const float2 c2 = *reinterpret_cast<const float2*>(cs_t + bl * kMaxCols + g * 8);
    const float u0 = dA * static_cast<float>(t1[g][0] - 32 * (r0[0] + 128 * r1[0]));
    const float u1 = dA * static_cast<float>(t1[g][1] - 32 * (r0[1] + 128 * r1[1]));
    const float u2 = dB * static_cast<float>(t1[g][2] - 32 * (r0[2] + 128 * r1[2]));
    const float u3 = dB * static_cast<float>(t1[g][3] - 32 * (r0[3] + 128 * r1[3]));
    o[g][0] = fmaf(c2.x, u0, o[g][0]);
    o[g][1] = fmaf(c2.y, u1, o[g][1]);
    o[g][2] = fmaf(c2.x, u2, o[g][2]);
    o[g][3] = fmaf(c2.y, u3, o[g][3]);
  }
}

struct alignas(64) Q6KMaps {
  CUtensorMap even[kMaxGroup], odd[kMaxGroup];
};

// A CTA works through the tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the launch's tile
// list, all on split chunk blockIdx.y of k (see gemv_mma.cu).
// SETS consumer warp sets (2, or 4 where each warp's chain of blocks would otherwise be long on
// a mostly idle SM): set s takes the chunks j = s (mod SETS) of the CTA's sequence.
// OUT: what follows the sums (staged_common.cuh: kOutGeneral, kOutPlain, kOutRanks); ONE: one
// weight tensor and one tile per CTA (tile loop and target choice compiled out).
template <int NCG, int SETS, bool ONE, int OUT, bool PRO>
__global__ void __launch_bounds__((SETS * 4 + 1) * 32, SETS == 2 ? 2 : 1)
gemv_q6k_staged_kernel(const __grid_constant__ Q6KMaps maps, const StagedParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kConsumerWarps = SETS * p.rgs, kConsumerThreads = kConsumerWarps * 32;
  const int kTileRows = 16 * p.rgs, kHalfBytes = p.rgs * kGroupHalfBytes, kStageBytes = 2 * kHalfBytes;
  unsigned char* act = smem + static_cast<size_t>(p.stages) * kStageBytes;
  unsigned char* sums = act + static_cast<size_t>(p.per) * p.ncols * 256;
  float* cs = reinterpret_cast<float*>(sums + static_cast<size_t>(p.per) * p.ncols * 2 * kGroups);
  float* xchg = cs + static_cast<size_t>(p.per) * kMaxCols;  // [SETS - 1][row groups][32 lanes][NCG*4]
  float* outbuf = xchg + (SETS - 1) * p.rgs * 32 * NCG * 4;  // [tile rows][NCG*8]
  uint64_t* full = reinterpret_cast<uint64_t*>(outbuf + kTileRows * NCG * 8);
  uint64_t* empty = full + p.stages;
  const unsigned char* zero_page = reinterpret_cast<const unsigned char*>(empty + p.stages);  // 16 zero bytes
  unsigned int* s_words = reinterpret_cast<unsigned int*>(empty + p.stages) + 4;              // [0] flag, [1] epoch
  // cluster split: arrival barriers and receive buffers of the chunk-0 CTA, one per tile of the CTA
  uint64_t* recv_bar = empty + p.stages + 4;
  float* rms_gain = reinterpret_cast<float*>(empty + p.stages + 8);  // [m] row gains of kProRmsNormLate
  float* recv = reinterpret_cast<float*>(empty + p.stages + 12);
  const bool clustered = TSR_CLUSTER_SPLIT != 0 && OUT == kOutGeneral && p.split_mode == kSplitCluster && gridDim.y > 1;
  const int b0 = blockIdx.y * p.per;
  // Stages cover block pairs (2j, 2j+1) of the row; pairs that straddle the
  // ends of this CTA's split chunk are loaded whole and half of them skipped.
  const int pair0 = b0 >> 1;
  const int nchunks = ((b0 + p.per + 1) >> 1) - pair0;
  const int my_tiles = ONE ? 1
                            : (p.total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                                  static_cast<int>(gridDim.x);
  const int total_chunks = my_tiles * nchunks;
  const bool producer = (tid == kConsumerThreads);

  if (tid < 4) reinterpret_cast<uint32_t*>(empty + p.stages)[tid] = 0u;
  if (producer) {
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < p.ntargets) {
        tma_prefetch_descriptor(&maps.even[g]);
        tma_prefetch_descriptor(&maps.odd[g]);
      }
    }
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], p.rgs);
    }
    if (clustered)
      for (int t = 0; t < kClusterTiles; ++t) mbar_init(&recv_bar[t], gridDim.y - 1);
    mbar_fence_init();
  }
  __syncthreads();
#if TSR_CLUSTER_SPLIT
  // no CTA of the cluster signals a peer's barrier before that peer has initialised it
  if (clustered) cluster_sync_all();
#endif

  // The producer walks the CTA's chunk sequence (tile after tile, pair after pair) with a
  // cursor: maps, first row and the odd map's shift change only when a tile begins.
  // Window of a chunk: starts at the 16-byte boundary at or below the pair, in
  // the byte space of each map (the odd map's base lies odd_shift bytes below
  // the first odd row).  Coordinates are in u64 units and even: 16-byte rule.
  int p_it = 0, p_c = 0, p_row0 = 0, p_shift = 0;
  const CUtensorMap* p_even = &maps.even[0];
  const CUtensorMap* p_odd = &maps.odd[0];
  auto issue_next = [&](int slot) {
    if (ONE) {
      p_row0 = blockIdx.x * kTileRows;
      p_shift = p.tgt[0].aux;
    } else if (p_c == 0) {
      const int tile = blockIdx.x + p_it * gridDim.x;
      const int g = target_of_tile(p, tile);
      const StagedTarget tgt = target_by_index(p, g);
      p_row0 = (tile - tgt.tile_begin) * kTileRows;
      p_shift = tgt.aux;
      p_even = map_by_index(maps.even, g);
      p_odd = map_by_index(maps.odd, g);
    }
    const uint32_t begin = static_cast<uint32_t>(pair0 + p_c) * kChunkBytes;
    unsigned char* dst = smem + static_cast<size_t>(slot) * kStageBytes;
    mbar_expect_tx(&full[slot], kStageBytes);
    tma_load_2d(dst, p_even, static_cast<int>((begin >> 4) * 2), p_row0 >> 1, &full[slot]);
    tma_load_2d(dst + kHalfBytes, p_odd, static_cast<int>(((begin + p_shift) >> 4) * 2), p_row0 >> 1, &full[slot]);
    if (++p_c == nchunks) {
      p_c = 0;
      ++p_it;
    }
  };
  auto prologue = [&]() {
    if (producer) {
      const int first = total_chunks < p.stages ? total_chunks : p.stages;
      for (int j = 0; j < first; ++j) issue_next(j);
    }
  };
  if (p.pdl) {
    // Weights are not written by the kernel ahead of us (the launcher checked):
    // start their prefetch; the wait for that kernel's results is inside the staging.
    prologue();
  }
  auto deferred_prologue = [&]() {
    if (!p.pdl) prologue();
  };
  if (!(p.debug & 1)) {
    stage_activations<kGroups, PRO>(p, b0 * kBlockElems, act, sums, cs, xchg, deferred_prologue);
  } else {
    if (p.pdl) pdl_wait();
    deferred_prologue();
  }
  if (OUT != kOutPlain && tid == 0 && p.tp.world > 1) s_words[1] = tp_call_epoch(p.tp);  // the stream's earlier work is complete here
  __syncthreads();
  if (OUT != kOutPlain && p.tp.world > 1 && warp < kConsumerWarps) {
    const size_t cta = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    tp_reset_previous(p.tp, s_words[1], cta * kConsumerThreads + tid,
                      static_cast<size_t>(gridDim.x) * gridDim.y * kConsumerThreads);
  }

  const bool late_gain = PRO && p.pro == kProRmsNormLate;
  if (late_gain && warp < kConsumerWarps) rms_late_gain(p, xchg, rms_gain, tid, kConsumerThreads);

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      RingCursor<SETS> cursor;
      cursor.start_after_fill(p.stages);
      for (int j = p.stages; j < total_chunks; ++j) {
        const RingUse use = cursor.next();
        if (!mbar_wait(&empty[use.slot], (use.round & 1) ^ 1, &g_q6k_wait_timeouts)) break;
        issue_next(use.slot);
      }
    }
    return;
  }

  const unsigned int epoch = s_words[1];
  const int gid = lane >> 2, tig = lane & 3;
  const int bx = warp / p.rgs, rg = warp - bx * p.rgs;  // warp set bx takes chunks j = bx (mod SETS)
  // A warp covers 16 consecutive rows: the thread's MMA rows gid and gid + 8 are
  // the even row 2e and the odd row 2e + 1 of pair e = 8 rg + gid.
  const int pair = rg * 8 + gid;
  const int rowA = 2 * pair;
  ThreadCtx tc[NCG];
#pragma unroll
  for (int g = 0; g < NCG; ++g) {
    const int col = g * 8 + gid;
    const bool valid = col < p.ncols;
    tc[g].act_t = valid ? act + col * 32 + tig * 4 : zero_page;
    tc[g].act_sb = valid ? p.ncols * 32 : 0;
    tc[g].act_blk = tc[g].act_sb * 8;
    tc[g].sum_t = valid ? sums + col * kGroups + tig * 4 : zero_page;
    tc[g].sum_plane = valid ? p.ncols * kGroups : 0;
    tc[g].sum_blk = tc[g].sum_plane * 2;
  }
  const float* cs_t = cs + 2 * tig;  // this thread's two columns of a group

  // this set's ring slots bx, bx + SETS, ... in turn (see ring_use)
  const int owned = (p.stages - bx + SETS - 1) / SETS;
  int ring_idx = 0, ring_round = 0;
  int j = bx;           // next chunk of this set in the CTA's sequence
  bool failed = false;  // a bounded wait gave up: skip the remaining waits, keep the barriers
  for (int it = 0; it < my_tiles; ++it) {
    const int tile = blockIdx.x + it * gridDim.x;
    const StagedTarget tg = ONE ? p.tgt[0] : target_by_index(p, target_of_tile(p, tile));
    const int row0 = ONE ? static_cast<int>(blockIdx.x) * kTileRows : (tile - tg.tile_begin) * kTileRows;
    const int odd_shift = tg.aux;
    float o[NCG][4];
#pragma unroll
    for (int g = 0; g < NCG; ++g)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[g][e] = 0.0f;

    const int jbase = it * nchunks, jend = jbase + nchunks;
    for (; j < jend && !failed; j += SETS) {
      const int c = j - jbase;
      const int slot = bx + SETS * ring_idx;
      if (!mbar_wait(&full[slot], ring_round & 1, &g_q6k_wait_timeouts)) {
        failed = true;
        break;
      }
      const uint32_t begin = static_cast<uint32_t>(pair0 + c) * kChunkBytes;
      const unsigned char* stage = smem + static_cast<size_t>(slot) * kStageBytes + pair * kRowPitch;
      const unsigned char* sa = stage + (begin & 15u);
      const unsigned char* sb = stage + kHalfBytes + ((begin + odd_shift) & 15u);
      const int bl = 2 * (pair0 + c) - b0;  // block index inside the split chunk: -1 for a straddling pair
      if (!(p.debug & 2)) {
        if (bl >= 0) q6k_block<false, NCG>(sa, sb, tig, bl, tc, cs_t, o);
        if (bl + 1 < p.per)
          q6k_block<true, NCG>(sa + kQ6KBlockBytes, sb + kQ6KBlockBytes, tig, bl + 1, tc, cs_t, o);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);
      if (++ring_idx == owned) {
        ring_idx = 0;
        ++ring_round;
      }
    }

    if (it == my_tiles - 1) pdl_trigger();  // the next launch may come in under this CTA's epilogue
    // The warps of a row group (one per set) add their partial sums; the digit
    // columns of each activation row are then combined through shared memory.
    if (bx > 0) {
#pragma unroll
      for (int g = 0; g < NCG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) xchg[((((bx - 1) * p.rgs + rg) * 32 + lane) * NCG + g) * 4 + e] = o[g][e];
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerThreads) : "memory");
    if (bx == 0) {
#pragma unroll
      for (int g = 0; g < NCG; ++g) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = g * 8 + 2 * tig + (e & 1);
          const int rr = rowA + (e >> 1);  // MMA row + 8 is the odd row of the pair
          float v = o[g][e];
#pragma unroll
          for (int sx = 0; sx < SETS - 1; ++sx) v += xchg[(((sx * p.rgs + rg) * 32 + lane) * NCG + g) * 4 + e];
          if (col < p.ncols) outbuf[rr * (NCG * 8) + col] = v;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerThreads) : "memory");
    if (OUT == kOutPlain) {
      // chunk y of k -> region y of the output (one region when k is not split)
      float* cout = tg.c + static_cast<size_t>(blockIdx.y) * p.m * tg.n;
      for (int idx = tid; idx < p.m * kTileRows; idx += kConsumerThreads) {
        const int i = idx / kTileRows, rr = idx - i * kTileRows;
        if (row0 + rr < tg.n) {
          float v = 0.0f;
          for (int t = p.terms - 1; t >= 0; --t) v += outbuf[rr * (NCG * 8) + i * p.terms + t];
          if (late_gain) v *= rms_gain[i];
          cout[static_cast<size_t>(i) * tg.n + row0 + rr] = v;
          if (tg.add_out != nullptr) {  // residual folded in (k is not split when there is one)
            const size_t e = static_cast<size_t>(i) * tg.n + row0 + rr;
            tg.add_out[e] = tg.add_src[e] + v;
          }
        }
      }
      continue;
    }
    if (OUT == kOutRanks) {
      // every thread sends its values to all ranks, then waits for the same elements of all
      // ranks in its own slots and adds them in rank order (tp_device.cuh)
      const size_t mine = tp_slot_offset(p.tp, epoch, p.tp.rank);
      for (int idx = tid; idx < p.m * kTileRows; idx += kConsumerThreads) {
        const int i = idx / kTileRows, rr = idx - i * kTileRows;
        if (row0 + rr < tg.n) {
          float v = 0.0f;
          for (int t = p.terms - 1; t >= 0; --t) v += outbuf[rr * (NCG * 8) + i * p.terms + t];
          if (late_gain) v *= rms_gain[i];
          tp_push(p.tp, mine + static_cast<size_t>(i) * tg.n + row0 + rr, v);
        }
      }
      for (int idx = tid; idx < p.m * kTileRows; idx += kConsumerThreads) {
        const int i = idx / kTileRows, rr = idx - i * kTileRows;
        if (row0 + rr < tg.n) {
          const size_t e = static_cast<size_t>(i) * tg.n + row0 + rr;
          const float v = tp_wait_sum(p.tp, epoch, e);
          tg.c[e] = v;
          if (tg.add_out != nullptr) tg.add_out[e] = tg.add_src[e] + v;
        }
      }
      continue;
    }
    finish_tile(p, tg, tile, row0, kTileRows, blockIdx.y, gridDim.y, epoch, tid, kConsumerThreads, s_words,
                it, recv_bar, recv, &g_q6k_wait_timeouts,
                [&](int i, int rr) {
                  float v = 0.0f;
                  for (int t = p.terms - 1; t >= 0; --t) v += outbuf[rr * (NCG * 8) + i * p.terms + t];
                  return late_gain ? v * rms_gain[i] : v;
                });
  }
  if (late_gain) rms_late_write(p, rms_gain, blockIdx.x, gridDim.x, tid, kConsumerThreads);
  if (OUT != kOutPlain && p.tp.world > 1) {
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerThreads) : "memory");  // every thread's share of the reset is done
    if (tid == 0) tp_cta_leaves(p.tp, epoch, gridDim.x * gridDim.y, static_cast<unsigned int>(p.m) * p.tgt[0].n);
  }
}

// ---- tensor-map cache: the pair of maps depends only on (base, rows, blocks per row, box rows)
struct MapKey {
  const void* base;
  uint64_t n, nb;
  int rgs;
  bool operator==(const MapKey& o) const { return base == o.base && n == o.n && nb == o.nb && rgs == o.rgs; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (k.n * 0x9E3779B97F4A7C15ull) ^ (k.nb << 40) ^
           (static_cast<size_t>(k.rgs) << 60);
  }
};
struct MapPair {
  CUtensorMap even, odd;
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, MapPair, MapKeyHash> g_maps;

int q6k_tensor_maps(const void* w, uint64_t n, uint64_t nb, int rgs, MapPair* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{w, n, nb, rgs};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return kOk;
  }
  const uint64_t row_bytes = nb * kQ6KBlockBytes;  // a multiple of 8
  const uint64_t shift = row_bytes & 15u;          // 0 or 8
  const uint64_t strides[1] = {2 * row_bytes};
  const uint32_t box[2] = {kWindowWords, static_cast<uint32_t>(8 * rgs)};
  // Inner extents end with the row: a window that runs past it reads zeros,
  // never bytes beyond the allocation.
  const uint64_t dims_even[2] = {row_bytes / 8, (n + 1) / 2};
  const uint64_t dims_odd[2] = {(row_bytes + shift) / 8, n / 2};
  MapPair pair;
  int rc = encode_tensor_map(&pair.even, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, w, dims_even, strides, box);
  if (rc != kOk) return rc;
  rc = encode_tensor_map(&pair.odd, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2,
                         static_cast<const unsigned char*>(w) + row_bytes - shift, dims_odd, strides, box);
  if (rc != kOk) return rc;
  if (g_maps.size() > 65536) g_maps.clear();
  g_maps.emplace(key, pair);
  *out = pair;
  return kOk;
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}

template <int NCG, int SETS>
int launch_group_q6k(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                     const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro,
                     double* cost_only) {
  const uint64_t nb = k / kBlockElems;
  const int terms = m <= 2 ? 3 : 2;
  const int ncols = static_cast<int>(m) * terms;
  auto fixed = [&](int rgs, uint64_t per) -> size_t {
    // receive buffers of a cluster split: one per tile of the CTA and chunk beyond the first
    const uint64_t chunks = per != 0 ? nb / per : 1;
    const size_t recv = caller_split == 0 && chunks > 1 ? kClusterTiles * (chunks - 1) * m * 16 * rgs * 4 : 0;
    return per * ncols * (256 + 2 * kGroups) + per * kMaxCols * 4 + (SETS - 1) * rgs * 32 * NCG * 4 * 4 +
           16 * rgs * NCG * 8 * 4 + 2 * 8 * 16 + 160 + recv;
  };
  auto stage_bytes = [](int rgs) -> size_t { return static_cast<size_t>(rgs) * 2 * kGroupHalfBytes; };
  auto chunks_of = [](uint64_t per) -> uint64_t { return per / 2 + 1; };
  static const int regs = kernel_registers(gemv_q6k_staged_kernel<NCG, SETS, false, kOutGeneral, true>);
  uint64_t rows[kMaxGroup];
  for (int i = 0; i < count; ++i) rows[i] = t[i].n;
  GroupPlan plan;
  if (!plan_group_cached(200 + NCG * 10 + SETS, rows, count, nb, static_cast<int>(m), caller_split, SETS, 0, regs, 8, 0.85, fixed, stage_bytes, chunks_of, &plan))
    return kUnsupportedFeature;
  if (plan.cluster) {
    // the cluster must be launchable (and, with ranks waiting on one another, all of the
    // launch's clusters resident at once); else the chunks meet through global memory
    if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&gemv_q6k_staged_kernel<NCG, SETS, false, kOutGeneral, true>), kMaxSmem)) return rc;
    const int fit = max_active_clusters(gemv_q6k_staged_kernel<NCG, SETS, false, kOutGeneral, true>, (SETS * plan.rgs + 1) * 32, plan.smem, plan.split);
    const bool with_ranks = tp != nullptr && tp->world > 1;
    if (fit < 1 || (with_ranks && fit < plan.grid_x)) {
      if (!plan_group_cached(200 + NCG * 10 + SETS, rows, count, nb, static_cast<int>(m), caller_split, SETS, 0, regs, 8, 0.85, fixed, stage_bytes, chunks_of, &plan, false))
        return kUnsupportedFeature;
    }
  }
  if (cost_only != nullptr) {
    *cost_only = plan.cost;
    return kOk;
  }
  const int forced = env_int("TSR_STAGES", 0);
  if (forced >= SETS && forced <= 16 &&
      fixed(plan.rgs, nb / plan.split) + forced * stage_bytes(plan.rgs) <= static_cast<size_t>(kMaxSmem)) {
    plan.stages = forced;
    plan.smem = fixed(plan.rgs, nb / plan.split) + forced * stage_bytes(plan.rgs);
  }
  if (plan.smem > static_cast<size_t>(kMaxSmem)) return kUnsupportedFeature;

  StagedParams p{};
  p.a = a;
  p.m = static_cast<int>(m);
  p.k = static_cast<int>(k);
  p.per = static_cast<int>(nb / plan.split);
  p.stages = plan.stages;
  p.terms = terms;
  p.ncols = ncols;
  p.debug = env_int("TSR_DEBUG", 0);
  p.rgs = plan.rgs;
  p.sets = SETS;
  p.ntargets = count;
  p.split_mode = caller_split != 0 ? kSplitCaller : (plan.cluster ? kSplitCluster : kSplitInLaunch);
  Q6KMaps maps{};
  const uint64_t th = 16u * plan.rgs;
  const int odd_shift = static_cast<int>((nb * kQ6KBlockBytes) & 15u);
  uint64_t tiles = 0;
  const void* reads[kMaxGroup];
  size_t read_bytes[kMaxGroup];
  const void* writes[2 * kMaxGroup + 1];
  size_t write_bytes[2 * kMaxGroup + 1];
  int nwrites = count;
  if (pro != nullptr) {
    p.a_bf16 = pro->bf16_in ? 1 : 0;
    p.c_bf16 = pro->bf16_out ? 1 : 0;
  }
  if (pro != nullptr && pro->kind != kProNone) {
    p.pro = pro->kind;
    p.eps = pro->eps;
    p.a2 = pro->other;
    p.a_out = pro->out;
    if (pro->out != nullptr) {
      writes[nwrites] = pro->out;
      write_bytes[nwrites++] = m * k * 4;
    }
  }
  for (int i = 0; i < count; ++i) {
    p.tgt[i] = StagedTarget{t[i].c, static_cast<int>(t[i].n), static_cast<int>(tiles), odd_shift, t[i].add_src, t[i].add_out};
    if (t[i].add_out != nullptr) {
      writes[nwrites] = t[i].add_out;
      write_bytes[nwrites++] = m * t[i].n * 4;
    }
    tiles += (t[i].n + th - 1) / th;
    MapPair pair;
    if (int rc = q6k_tensor_maps(t[i].w, t[i].n, nb, plan.rgs, &pair)) return rc;
    maps.even[i] = pair.even;
    maps.odd[i] = pair.odd;
    reads[i] = t[i].w;
    read_bytes[i] = t[i].n * nb * kQ6KBlockBytes;
    writes[i] = t[i].c;
    write_bytes[i] = (caller_split != 0 ? caller_split : 1) * m * t[i].n * 4;
  }
  p.total_tiles = static_cast<int>(tiles);
  if (p.split_mode == kSplitInLaunch && plan.split > 1) {
    const size_t need = static_cast<size_t>(plan.split) * tiles * m * th;
    if (scratch == nullptr || scratch->part == nullptr || need > scratch->part_floats || tiles > scratch->ntickets)
      return kUnsupportedFeature;
    p.part = scratch->part;
    p.tickets = scratch->tickets;
  }
  if (tp != nullptr && tp->world > 1) {
    if (m * t[0].n > tp->capacity || count != 1 || p.split_mode == kSplitCaller) return kUnsupportedFeature;
    // every CTA of the launch must be resident at once: a tile waits for its peers' values
    if (static_cast<uint64_t>(plan.grid_x) * plan.split > static_cast<uint64_t>(device_sms()) * plan.occ)
      return kUnsupportedFeature;
    p.tp = *tp;
  } else {
    p.tp.world = 1;
  }
  // the trimmed variants where the general output stage is not needed (TSR_LEAN=0: experiments);
  // those that also fold an elementwise step or read bf16 exist for one column group only
  const bool trim = env_int("TSR_LEAN", 1) != 0 && p.c_bf16 == 0;
  bool has_add = false;
  for (int i = 0; i < count; ++i) has_add = has_add || t[i].add_out != nullptr;
  // rmsnorm where every CTA stages whole rows: the gain multiplies the sums instead of the activations
  if (p.pro == kProRmsNorm && plan.split == 1 && p.a_bf16 == 0 &&
      m * (nb + 1) <= static_cast<uint64_t>(128) * SETS * plan.rgs * NCG && env_int("TSR_RMS_LATE", 1) != 0)
    p.pro = kProRmsNormLate;
  const bool has_pro = p.pro != kProNone || p.a_bf16 != 0;
  const bool plain = trim && p.tp.world == 1 && (plan.split == 1 || (p.split_mode == kSplitCaller && !has_add));
  const bool ranks = trim && p.tp.world > 1 && plan.split == 1;
  const bool one = count == 1 && static_cast<uint64_t>(plan.grid_x) == tiles;
  auto kernel = gemv_q6k_staged_kernel<NCG, SETS, false, kOutGeneral, true>;
  if (plain && !has_pro)
    kernel = one ? gemv_q6k_staged_kernel<NCG, SETS, true, kOutPlain, false> : gemv_q6k_staged_kernel<NCG, SETS, false, kOutPlain, false>;
  else if (ranks && !has_pro)
    kernel = one ? gemv_q6k_staged_kernel<NCG, SETS, true, kOutRanks, false> : gemv_q6k_staged_kernel<NCG, SETS, false, kOutRanks, false>;
  if constexpr (NCG == 1) {
    if (plain && has_pro)
      kernel = one ? gemv_q6k_staged_kernel<NCG, SETS, true, kOutPlain, true> : gemv_q6k_staged_kernel<NCG, SETS, false, kOutPlain, true>;
    else if (ranks && has_pro && one)
      kernel = gemv_q6k_staged_kernel<NCG, SETS, true, kOutRanks, true>;
  }
  if (kernel != gemv_q6k_staged_kernel<NCG, SETS, false, kOutGeneral, true> && p.tp.world == 1) p.split_mode = kSplitCaller;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxSmem)) return rc;
  const dim3 grid(static_cast<unsigned>(plan.grid_x), static_cast<unsigned>(plan.split));
  p.pdl = pdl_allowed_ranges(st, reads, read_bytes, count, writes, write_bytes, nwrites) ? 1 : 0;
  {
    const int mode = env_int("TSR_PDL_MODE", 1);  // experiments: which launches may start before their predecessor ends
    if (mode == 2 && plan.occ < 2) p.pdl = 0;
    if (mode == 3 && plan.sets != 4) p.pdl = 0;
  }
  launch_kernel_cluster_y(kernel, grid, dim3((SETS * plan.rgs + 1) * 32), plan.smem, st,
                          p.pdl != 0, plan.cluster ? static_cast<unsigned>(plan.split) : 1u, maps, p);
  return check_launch();
}

}  // namespace

// Returns kUnsupportedFeature when the launch is outside what the staged
// kernel covers; the caller then uses the general warp-per-row family.
int staged_group_q6k(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                     const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro) {
  const uint64_t nb = k / kBlockElems;
  if (m > 8 || count < 1 || count > kMaxGroup || nb % 4 != 0 || env_int("TSR_DISABLE_STAGED", 0))
    return kUnsupportedFeature;
  if (caller_split != 0) {
    if (pro != nullptr && (pro->kind != kProNone || pro->bf16_in || pro->bf16_out)) return kUnsupportedFeature;
    for (int i = 0; i < count; ++i)
      if (t[i].add_out != nullptr) return kUnsupportedFeature;
  }
  // Rows must be 8-byte aligned inside a 16-byte aligned matrix, and there must be an odd row.
  for (int i = 0; i < count; ++i)
    if (t[i].n < 2 || (reinterpret_cast<uintptr_t>(t[i].w) & 15u)) return kUnsupportedFeature;
  const int ncols = static_cast<int>(m) * (m <= 2 ? 3 : 2);
  // two consumer sets, or four when the model says the warps' own chains of blocks set the time
  auto run = [&](auto ncg) -> int {
    constexpr int kNcg = decltype(ncg)::value;
    double c2 = 0.0, c4 = 0.0;
    const int r2 = launch_group_q6k<kNcg, 2>(a, t, count, m, k, caller_split, scratch, tp, st, pro, &c2);
    const int r4 = launch_group_q6k<kNcg, 4>(a, t, count, m, k, caller_split, scratch, tp, st, pro, &c4);
    const int forced_sets = env_int("TSR_SETS", 0);
    const bool four = forced_sets == 4 ? r4 == kOk : forced_sets == 2 ? r2 != kOk && r4 == kOk
                                                                      : r4 == kOk && (r2 != kOk || c4 + 0.3 < c2);
    if (four) return launch_group_q6k<kNcg, 4>(a, t, count, m, k, caller_split, scratch, tp, st, pro, nullptr);
    if (r2 != kOk) return r2;
    return launch_group_q6k<kNcg, 2>(a, t, count, m, k, caller_split, scratch, tp, st, pro, nullptr);
  };
  if (ncols <= 8) return run(std::integral_constant<int, 1>{});
  return run(std::integral_constant<int, 2>{});
}

int staged_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    uint64_t split, cudaStream_t st) {
  const GroupTarget t{w, c, n};
  return staged_group_q6k(a, &t, 1, m, k, split, nullptr, nullptr, st);
}

int staged_q6k_set_error_word(unsigned int* word) { return set_host_error_word(word); }

int staged_q6k_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_q6k_wait_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}

}  // namespace tsr
