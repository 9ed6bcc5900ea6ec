// Staged tensor-pipe GEMV for Q4_K weights (m = 1..8 activation rows).
//
// Data path, per CTA (one tile of 16..64 rows of W, one split chunk of k):
//   HBM --TMA 3-D box (tile rows x 2 blocks x 144 B per stage)--> shared
//   memory ring --LDS.64 per thread--> packed nibbles --one LOP3 per four
//   weights--> u8 A fragments --mma.sync m16n8k32 (s32 accumulate)--> registers
//   --per-sub-block integer scale, per-block fp32 scale--> C.
// Tile height, CTAs per SM and ring depth come from staged_common.cuh::plan_staged.
//
// Weights are the A operand (16 weight rows per warp), activations the B
// operand.  Each 256-element block of an fp32 activation row is expanded,
// once per CTA, into signed base-256 int8 "digit" columns
// a ~= unit*(q1*65536 + q2*256 + q3) (three digits for m <= 2, two above), so
// the dot products are exact integer arithmetic and the only rounding is the
// <= 1.2e-7 (three digits) or <= 3.1e-5 (two digits) quantisation of the
// activation relative to the largest magnitude of its block.  One MMA covers
// exactly one 32-element Q4_K sub-block, whose 6-bit scale multiplies the
// integer partial sum; the fp16 super-block scale d is applied in fp32 once
// per block.  The -dmin*mn*sum(a) term of the format
// (src/core/numerics/quant.cpp:656-675 of the reference: w = d*sc*q - dmin*mn)
// is two more MMAs per block against per-sub-block activation digit sums.
//
// Shared-memory reads are conflict free: the box row pitch (2 * 144 = 288 B)
// is 32 mod 128, so the sixteen lanes of an LDS.64 phase (four rows x four
// 8-byte pieces) cover all 32 banks once.
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

__device__ unsigned int g_wait_timeouts = 0;

namespace {

// A CTA owns 16 * rgs rows of W (rgs = 1..4 row groups, chosen per launch) and
// runs two sets of rgs consumer warps; the sets alternate between stages.
constexpr int kBoxBlocks = 2;   // Q4_K blocks per box row (pitch 288 B)
constexpr int kChunkBlocks = kBoxBlocks;
constexpr int kRowPitch = kBoxBlocks * kQ4KBlockBytes;
constexpr int kGroupBytes = 16 * kRowPitch;  // one row group of one stage: 4608

using namespace staged;

struct alignas(64) Q4KMaps {
  CUtensorMap m[kMaxGroup];
};

// SETS consumer warp sets (2, or 4 for launches whose warps would otherwise each walk a long
// chain of chunks on a mostly idle SM: the sets split the chunks of k among them).
// A CTA works through the tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the launch's tile
// list, all on split chunk blockIdx.y of k: the activations are staged once, and the weight
// ring keeps streaming across tile boundaries.
// OUT selects what follows the sums.  kOutGeneral: everything finish_tile offers (the split of k
// added inside the launch, ranks, residual, bf16).  kOutPlain: any split of k is left to the
// caller and nothing follows (fp32 store).  kOutRanks: the sum over tensor-parallel ranks and
// an optional residual, k not split.  The trimmed forms exist because the general stage costs
// launches that never use it: the 27B-class step went from 4.75 to 4.13 ms with kOutPlain.
// ONE (not with kOutGeneral): one weight tensor and one tile per CTA, so the tile loop and the
// choice of target are compiled out as well.
template <int NCG, int SETS, bool ONE, int OUT, bool PRO>
__global__ void __launch_bounds__((SETS * 4 + 1) * 32, SETS == 2 ? 2 : 1)
gemv_q4k_staged_kernel(const __grid_constant__ Q4KMaps maps, const StagedParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kConsumerWarps = SETS * p.rgs, kConsumerThreads = kConsumerWarps * 32;
  const int kTileRows = 16 * p.rgs, kStageBytes = p.rgs * kGroupBytes;
  const int nchunks = (p.per + kChunkBlocks - 1) / kChunkBlocks;
  const int nblk_pad = nchunks * kChunkBlocks;
  unsigned char* act = smem + static_cast<size_t>(p.stages) * kStageBytes;
  unsigned char* sums = act + static_cast<size_t>(nblk_pad) * p.ncols * 256;
  float* cs = reinterpret_cast<float*>(sums + static_cast<size_t>(nblk_pad) * p.ncols * 16);  // [block][kMaxCols]
  float* xchg = cs + static_cast<size_t>(nblk_pad) * kMaxCols;  // [SETS - 1][row groups][32 lanes][NCG*4]
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
  const int my_tiles = ONE ? 1
                            : (p.total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                                  static_cast<int>(gridDim.x);
  const int total_chunks = my_tiles * nchunks;
  const bool producer = (tid == kConsumerThreads);

  if (tid < 4) reinterpret_cast<uint32_t*>(empty + p.stages)[tid] = 0u;
  if (producer) {
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
      if (g < p.ntargets) tma_prefetch_descriptor(&maps.m[g]);
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
  // The producer walks the CTA's chunk sequence (tile after tile, chunk after chunk) with a
  // cursor: map and first row change only when a tile begins.
  int p_it = 0, p_c = 0, p_row0 = 0;
  const CUtensorMap* p_map = &maps.m[0];
  auto issue_next = [&](int slot) {
    if (ONE) {
      p_row0 = blockIdx.x * kTileRows;
    } else if (p_c == 0) {
      const int tile = blockIdx.x + p_it * gridDim.x;
      const int g = target_of_tile(p, tile);
      p_row0 = (tile - target_by_index(p, g).tile_begin) * kTileRows;
      p_map = map_by_index(maps.m, g);
    }
    unsigned char* dst = smem + static_cast<size_t>(slot) * kStageBytes;
    mbar_expect_tx(&full[slot], kStageBytes);
    tma_load_3d(dst, p_map, 0, b0 + p_c * kChunkBlocks, p_row0, &full[slot]);
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
    stage_activations<8, PRO>(p, b0 * kBlockElems, act, sums, cs, xchg, deferred_prologue);
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
        if (!mbar_wait(&empty[use.slot], (use.round & 1) ^ 1, &g_wait_timeouts)) break;
        issue_next(use.slot);
      }
    }
    return;
  }

  const unsigned int epoch = s_words[1];
  const int gid = lane >> 2, tig = lane & 3;
  const int bx = warp / p.rgs, rg = warp - bx * p.rgs;  // warp set bx takes chunks j = bx (mod SETS)
  const int rowA = rg * 16 + gid;
  constexpr uint32_t kNib = 0x0F0F0F0Fu, kHiNib = 0xF0F0F0F0u;

  // Per-thread fragment addresses.  A lane whose column does not exist reads
  // the zero page with zero strides, so the loop needs no predicates.
  const unsigned char* act_t[NCG];
  const unsigned char* sum_t[NCG];
  uint32_t act_sb[NCG], act_blk[NCG], sum_plane[NCG], sum_blk[NCG];
#pragma unroll
  for (int g = 0; g < NCG; ++g) {
    const int col = g * 8 + gid;
    const bool valid = col < p.ncols;
    act_t[g] = valid ? act + col * 32 + tig * 8 : zero_page;
    act_sb[g] = valid ? p.ncols * 32 : 0;
    act_blk[g] = act_sb[g] * 8;
    const bool sv = valid && tig < 2;
    sum_t[g] = sv ? sums + col * 8 + tig * 4 : zero_page;
    sum_plane[g] = sv ? p.ncols * 8 : 0;
    sum_blk[g] = sum_plane[g] * 2;
  }
  const uint32_t mask0 = tig == 0 ? 0xFFFFFFFFu : 0u, mask1 = tig == 1 ? 0xFFFFFFFFu : 0u;
  const float* cs_t = cs + 2 * tig;  // this thread's two columns of a group
  const uint32_t row_off = rowA * kRowPitch;

  // this set's ring slots bx, bx + SETS, ... in turn (see ring_use)
  const int owned = (p.stages - bx + SETS - 1) / SETS;
  int ring_idx = 0, ring_round = 0;
  int j = bx;           // next chunk of this set in the CTA's sequence
  bool failed = false;  // a bounded wait gave up: skip the remaining waits, keep the barriers
  for (int it = 0; it < my_tiles; ++it) {
    const int tile = blockIdx.x + it * gridDim.x;
    float o[NCG][4];
#pragma unroll
    for (int g = 0; g < NCG; ++g)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[g][e] = 0.0f;

    const int jbase = it * nchunks, jend = jbase + nchunks;
    for (; j < jend && !failed; j += SETS) {
      const int c = j - jbase;
      const int slot = bx + SETS * ring_idx;
      if (!mbar_wait(&full[slot], ring_round & 1, &g_wait_timeouts)) {
        failed = true;
        break;
      }
      const unsigned char* st = smem + static_cast<size_t>(slot) * kStageBytes + row_off;
      const int blocks_here = (p.debug & 2) ? 0 : min(kBoxBlocks, p.per - c * kChunkBlocks);
#pragma unroll
      for (int bi = 0; bi < kBoxBlocks; ++bi) {
        if (bi < blocks_here) {
          const int bl = c * kChunkBlocks + bi;
          const unsigned char* pa = st + bi * kQ4KBlockBytes;
          const unsigned char* pb = pa + 8 * kRowPitch;
          const uint4 ha = lds128(pa), hb = lds128(pb);
          // 6-bit scales and mins of the 8 sub-blocks as bytes (quant.cpp:58-70)
          const uint32_t scA[2] = {ha.y & 0x3F3F3F3Fu, (ha.w & kNib) | ((ha.y >> 2) & 0x30303030u)};
          const uint32_t mnA[2] = {ha.z & 0x3F3F3F3Fu, ((ha.w >> 4) & kNib) | ((ha.z >> 2) & 0x30303030u)};
          const uint32_t scB[2] = {hb.y & 0x3F3F3F3Fu, (hb.w & kNib) | ((hb.y >> 2) & 0x30303030u)};
          const uint32_t mnB[2] = {hb.z & 0x3F3F3F3Fu, ((hb.w >> 4) & kNib) | ((hb.z >> 2) & 0x30303030u)};

          // t1: low-nibble sub-blocks; t16: high-nibble sub-blocks, whose weights enter the MMA
          // as 16 q (the nibble masked in place, no shift); the 16 is taken out again below
          int t1[NCG][4], t16[NCG][4];
#pragma unroll
          for (int g = 0; g < NCG; ++g)
#pragma unroll
            for (int e = 0; e < 4; ++e) t1[g][e] = t16[g][e] = 0;

#pragma unroll
          for (int grp = 0; grp < 4; ++grp) {
            const uint2 qa = lds64(pa + 16 + 32 * grp + 8 * tig);
            const uint2 qb = lds64(pb + 16 + 32 * grp + 8 * tig);
            const int sclA = __byte_perm(scA[grp >> 1], 0, 0x4440 + 2 * (grp & 1));
            const int schA = __byte_perm(scA[grp >> 1], 0, 0x4441 + 2 * (grp & 1));
            const int sclB = __byte_perm(scB[grp >> 1], 0, 0x4440 + 2 * (grp & 1));
            const int schB = __byte_perm(scB[grp >> 1], 0, 0x4441 + 2 * (grp & 1));
#pragma unroll
            for (int g = 0; g < NCG; ++g) {
              const unsigned char* ab = act_t[g] + bl * act_blk[g];
              const uint2 fl = lds64(ab + (2 * grp) * act_sb[g]);
              const uint2 fh = lds64(ab + (2 * grp + 1) * act_sb[g]);
              int pl[4], ph[4];
              mma_u8s8_zero(pl, qa.x & kNib, qb.x & kNib, qa.y & kNib, qb.y & kNib, fl.x, fl.y);
              mma_u8s8_zero(ph, qa.x & kHiNib, qb.x & kHiNib, qa.y & kHiNib, qb.y & kHiNib, fh.x, fh.y);
              t1[g][0] += sclA * pl[0];
              t1[g][1] += sclA * pl[1];
              t1[g][2] += sclB * pl[2];
              t1[g][3] += sclB * pl[3];
              t16[g][0] += schA * ph[0];
              t16[g][1] += schA * ph[1];
              t16[g][2] += schB * ph[2];
              t16[g][3] += schB * ph[3];
            }
          }
          // min term: k slots 0..7 are the sub-blocks; lanes tig 0/1 hold mins 0..3 / 4..7
          const uint32_t am = (mnA[0] & mask0) | (mnA[1] & mask1);
          const uint32_t bm = (mnB[0] & mask0) | (mnB[1] & mask1);
          // the sums below are 16 x the block's integer dot product (all of them < 2^31): d / 16 is exact
          const float dA = fp16_bits_to_float(ha.x & 0xFFFFu) * 0.0625f, mA = fp16_bits_to_float(ha.x >> 16);
          const float dB = fp16_bits_to_float(hb.x & 0xFFFFu) * 0.0625f, mB = fp16_bits_to_float(hb.x >> 16);
#pragma unroll
          for (int g = 0; g < NCG; ++g) {
            const unsigned char* sp = sum_t[g] + bl * sum_blk[g];
            const uint32_t s0 = *reinterpret_cast<const uint32_t*>(sp);
            const uint32_t s1 = *reinterpret_cast<const uint32_t*>(sp + sum_plane[g]);
            int r0[4], r1[4];
            mma_u8s8_zero(r0, am, bm, 0u, 0u, s0, 0u);
            mma_u8s8_zero(r1, am, bm, 0u, 0u, s1, 0u);
            const float2 c2 = *reinterpret_cast<const float2*>(cs_t + bl * kMaxCols + g * 8);
            const float u0 = fmaf(dA, static_cast<float>(16 * t1[g][0] + t16[g][0]), -mA * static_cast<float>(r0[0] + 128 * r1[0]));
            const float u1 = fmaf(dA, static_cast<float>(16 * t1[g][1] + t16[g][1]), -mA * static_cast<float>(r0[1] + 128 * r1[1]));
            const float u2 = fmaf(dB, static_cast<float>(16 * t1[g][2] + t16[g][2]), -mB * static_cast<float>(r0[2] + 128 * r1[2]));
            const float u3 = fmaf(dB, static_cast<float>(16 * t1[g][3] + t16[g][3]), -mB * static_cast<float>(r0[3] + 128 * r1[3]));
            o[g][0] = fmaf(c2.x, u0, o[g][0]);
            o[g][1] = fmaf(c2.y, u1, o[g][1]);
            o[g][2] = fmaf(c2.x, u2, o[g][2]);
            o[g][3] = fmaf(c2.y, u3, o[g][3]);
          }
        }
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
          const int rr = rowA + (e >> 1) * 8;
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
      const StagedTarget tg = ONE ? p.tgt[0] : target_by_index(p, target_of_tile(p, tile));
      const int row0 = (ONE ? static_cast<int>(blockIdx.x) : tile - tg.tile_begin) * kTileRows;
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
      const StagedTarget tg = ONE ? p.tgt[0] : target_by_index(p, target_of_tile(p, tile));
      const int row0 = (ONE ? static_cast<int>(blockIdx.x) : tile - tg.tile_begin) * kTileRows;
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
    const StagedTarget tg = target_by_index(p, target_of_tile(p, tile));
    const int row0 = (tile - tg.tile_begin) * kTileRows;
    finish_tile(p, tg, tile, row0, kTileRows, blockIdx.y, gridDim.y, epoch, tid, kConsumerThreads, s_words,
                it, recv_bar, recv, &g_wait_timeouts,
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

// ---- tensor-map cache: a map depends only on (base, rows, blocks per row, box rows)
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
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int q4k_tensor_map(const void* w, uint64_t n, uint64_t nb, int rgs, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{w, n, nb, rgs};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return kOk;
  }
  // (18 x u64 = one 144-byte block, blocks of a row, rows)
  const uint64_t dims[3] = {18, nb, n};
  const uint64_t strides[2] = {kQ4KBlockBytes, nb * kQ4KBlockBytes};
  const uint32_t box[3] = {18, kBoxBlocks, static_cast<uint32_t>(16 * rgs)};
  CUtensorMap map;
  const int rc = encode_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, w, dims, strides, box);
  if (rc != kOk) return rc;
  if (g_maps.size() > 65536) g_maps.clear();
  g_maps.emplace(key, map);
  *out = map;
  return kOk;
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}

// Plans and issues one launch with SETS consumer sets; with `cost_only` the launch is planned
// but not issued, and its modelled time returned.
template <int NCG, int SETS>
int launch_group(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                 const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro,
                 double* cost_only) {
  const uint64_t nb = k / kBlockElems;
  const int terms = m <= 2 ? 3 : 2;
  const int ncols = static_cast<int>(m) * terms;
  auto chunks_of = [](uint64_t per) -> uint64_t { return (per + kChunkBlocks - 1) / kChunkBlocks; };
  auto fixed = [&](int rgs, uint64_t per) -> size_t {
    const uint64_t nblk_pad = chunks_of(per) * kChunkBlocks;
    // receive buffers of a cluster split: one per tile of the CTA and chunk beyond the first
        const uint64_t chunks = per != 0 ? nb / per : 1;
        const size_t recv = caller_split == 0 && chunks > 1 ? kClusterTiles * (chunks - 1) * m * 16 * rgs * 4 : 0;
    return nblk_pad * ncols * (256 + 16) + nblk_pad * kMaxCols * 4 + (SETS - 1) * rgs * 32 * NCG * 4 * 4 +
           16 * rgs * NCG * 8 * 4 + 2 * 8 * 16 + 160 + recv;
  };
  auto stage_bytes = [](int rgs) -> size_t { return static_cast<size_t>(rgs) * kGroupBytes; };
  static const int regs = kernel_registers(gemv_q4k_staged_kernel<NCG, SETS, false, kOutGeneral, true>);
  uint64_t rows[kMaxGroup];
  for (int i = 0; i < count; ++i) rows[i] = t[i].n;
  GroupPlan plan;
  if (!plan_group_cached(100 + NCG * 10 + SETS, rows, count, nb, static_cast<int>(m), caller_split, SETS, 0, regs, 12, 0.5, fixed, stage_bytes, chunks_of, &plan))
    return kUnsupportedFeature;
  if (plan.cluster) {
    // the cluster must be launchable (and, with ranks waiting on one another, all of the
    // launch's clusters resident at once); else the chunks meet through global memory
    if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&gemv_q4k_staged_kernel<NCG, SETS, false, kOutGeneral, true>), kMaxSmem)) return rc;
    const int fit = max_active_clusters(gemv_q4k_staged_kernel<NCG, SETS, false, kOutGeneral, true>, (SETS * plan.rgs + 1) * 32, plan.smem, plan.split);
    const bool with_ranks = tp != nullptr && tp->world > 1;
    if (fit < 1 || (with_ranks && fit < plan.grid_x)) {
      if (!plan_group_cached(100 + NCG * 10 + SETS, rows, count, nb, static_cast<int>(m), caller_split, SETS, 0, regs, 12, 0.5, fixed, stage_bytes, chunks_of, &plan, false))
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
  Q4KMaps maps{};
  const uint64_t th = 16u * plan.rgs;
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
    p.tgt[i] = StagedTarget{t[i].c, static_cast<int>(t[i].n), static_cast<int>(tiles), 0, t[i].add_src, t[i].add_out};
    if (t[i].add_out != nullptr) {
      writes[nwrites] = t[i].add_out;
      write_bytes[nwrites++] = m * t[i].n * 4;
    }
    tiles += (t[i].n + th - 1) / th;
    if (int rc = q4k_tensor_map(t[i].w, t[i].n, nb, plan.rgs, &maps.m[i])) return rc;
    reads[i] = t[i].w;
    read_bytes[i] = t[i].n * nb * kQ4KBlockBytes;
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
  auto kernel = gemv_q4k_staged_kernel<NCG, SETS, false, kOutGeneral, true>;
  if (plain && !has_pro)
    kernel = one ? gemv_q4k_staged_kernel<NCG, SETS, true, kOutPlain, false> : gemv_q4k_staged_kernel<NCG, SETS, false, kOutPlain, false>;
  else if (ranks && !has_pro)
    kernel = one ? gemv_q4k_staged_kernel<NCG, SETS, true, kOutRanks, false> : gemv_q4k_staged_kernel<NCG, SETS, false, kOutRanks, false>;
  if constexpr (NCG == 1) {
    if (plain && has_pro)
      kernel = one ? gemv_q4k_staged_kernel<NCG, SETS, true, kOutPlain, true> : gemv_q4k_staged_kernel<NCG, SETS, false, kOutPlain, true>;
    else if (ranks && has_pro && one)
      kernel = gemv_q4k_staged_kernel<NCG, SETS, true, kOutRanks, true>;
  }
  if (kernel != gemv_q4k_staged_kernel<NCG, SETS, false, kOutGeneral, true> && p.tp.world == 1) p.split_mode = kSplitCaller;
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

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      bool swizzle128) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeFn>(fn);
  });
  if (!encode) return kDeviceError;
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], e[5];
  for (uint32_t i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i + 1 < rank) s[i] = strides_bytes[i];
  }
  const CUresult r = encode(map, type, rank, const_cast<void*>(base), d, s, b, e,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kInvalidArgument;
}

// Returns kUnsupportedFeature when the launch is outside what the staged
// kernel covers; the caller then uses the general warp-per-row family.
// caller_split >= 1: chunk y of k goes to region y of each target (the caller
// adds the regions); caller_split == 0: the launch splits k as it sees fit and
// adds the chunks itself (needs `scratch` when it does split).
int staged_group_q4k(const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k, uint64_t caller_split,
                     const FusedScratch* scratch, const TpTail* tp, cudaStream_t st, const Prologue* pro) {
  if (m > 8 || count < 1 || count > kMaxGroup || env_int("TSR_DISABLE_STAGED", 0)) return kUnsupportedFeature;
  if (caller_split != 0) {
    if (pro != nullptr && (pro->kind != kProNone || pro->bf16_in || pro->bf16_out)) return kUnsupportedFeature;
    for (int i = 0; i < count; ++i)
      if (t[i].add_out != nullptr) return kUnsupportedFeature;
  }
  const int ncols = static_cast<int>(m) * (m <= 2 ? 3 : 2);
  // two consumer sets, or four when the model says the warps' own chains of chunks
  // (not the SM's throughput) set the time: few CTAs, long k
  auto run = [&](auto ncg) -> int {
    constexpr int kNcg = decltype(ncg)::value;
    double c2 = 0.0, c4 = 0.0;
    const int r2 = launch_group<kNcg, 2>(a, t, count, m, k, caller_split, scratch, tp, st, pro, &c2);
    const int r4 = launch_group<kNcg, 4>(a, t, count, m, k, caller_split, scratch, tp, st, pro, &c4);
    const int forced_sets = env_int("TSR_SETS", 0);
    const bool four = forced_sets == 4 ? r4 == kOk : forced_sets == 2 ? r2 != kOk && r4 == kOk
                                                                      : r4 == kOk && (r2 != kOk || c4 + 0.3 < c2);
    if (four) return launch_group<kNcg, 4>(a, t, count, m, k, caller_split, scratch, tp, st, pro, nullptr);
    if (r2 != kOk) return r2;
    return launch_group<kNcg, 2>(a, t, count, m, k, caller_split, scratch, tp, st, pro, nullptr);
  };
  if (ncols <= 8) return run(std::integral_constant<int, 1>{});
  return run(std::integral_constant<int, 2>{});
}

int staged_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    uint64_t split, cudaStream_t st) {
  const GroupTarget t{w, c, n};
  return staged_group_q4k(a, &t, 1, m, k, split, nullptr, nullptr, st);
}

int staged_set_error_word(unsigned int* word) { return set_host_error_word(word); }

int staged_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_wait_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}

}  // namespace tsr
