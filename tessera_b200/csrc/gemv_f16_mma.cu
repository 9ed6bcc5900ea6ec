// Staged tensor-pipe GEMV for MXFP4 and FP8 E4M3 weights (m = 1..8 activation rows).
//
// Same skeleton as the Q4_K kernel (gemv_mma.cu): one CTA per tile of 16..64
// weight rows, a TMA-fed ring of shared-memory stages, one producer thread,
// two sets of consumer warps that alternate between stages, weights as the A
// operand of mma.sync, activations as the B operand.  The arithmetic differs:
//   * Both formats convert to binary16 exactly with one cvt per two weights
//     (cvt.rn.f16x2.e2m1x2 / .e4m3x2), so the MMA is m16n8k16 f16 x f16 -> f32.
//   * An fp32 activation becomes two binary16 columns per row, hi = rn(v) and
//     lo = rn((v - hi) * 2^11) with v = x / unit and unit = block maximum / 1024
//     per 256-element block: 22 significant bits, every product exact in the
//     fp32 accumulator.
//   * MXFP4 (src/core/numerics/gemm.cpp:311-344 of the reference: rows of k/2
//     nibble bytes, low nibble the even element, then n x k/32 E8M0 scales):
//     the two MMAs of a 32-element scale block accumulate alone and the sum
//     is scaled by 2^(e-127) in fp32.  The scale bytes of a stage arrive by a
//     second small TMA box from the side table.
//   * FP8 (gemm.cpp:253-277: n x k bytes, one fp32 scale per row): the MMAs of
//     a 256-element block chain in the accumulator; the row scale multiplies
//     the final sum.
// Stages are [2 segments][rows][128 B] with the 128-byte swizzle, so the
// 4-byte fragment loads of eight rows hit eight different 16-byte pieces.
// When k * columns does not fit shared memory the activations are staged in
// phases of `pblocks` blocks; the weight ring keeps streaming across phases.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "codec.cuh"
#include "launch.h"
#include "pipeline.cuh"
#include "staged_common.cuh"

namespace tsr {

__device__ unsigned int g_f16_wait_timeouts = 0;

namespace {

using namespace staged;

constexpr int kFmtMxfp4 = 0, kFmtFp8 = 1;
constexpr int kSegBytes = 128;
constexpr int kGroupStageBytes = 2 * 16 * kSegBytes;  // one 16-row group of one stage: 4096
constexpr int kGroupScaleBytes = 16 * 16;             // MXFP4: 16 scale bytes per row and stage
constexpr float kLoScale = 2048.0f;

struct F16Params {
  const float* a;
  float* c;
  const float* row_scale;  // FP8 only
  int m, n, k;
  int nblocks;  // k / 256
  int pblocks;  // activation blocks staged per phase
  int stages;   // ring depth
  int ncols;    // 2 * m
  int pdl;      // launched as a programmatic dependent
  int rgs;      // 16-row groups per CTA
  int ksplit;   // CTAs of a cluster that share a row tile, each with `cper` consecutive chunks
  int cper;
};

template <int FMT>
struct Fmt;
template <>
struct Fmt<kFmtMxfp4> {
  static constexpr int kChunkElems = 512;  // 2 x 128 bytes of nibbles per row
  static constexpr int kGroup = 32;        // activation halves stored per (k group, column)
};
template <>
struct Fmt<kFmtFp8> {
  static constexpr int kChunkElems = 256;
  static constexpr int kGroup = 16;
};

__device__ __forceinline__ uint32_t lds32(const unsigned char* p) {
  return *reinterpret_cast<const uint32_t*>(p);
}

// Four E2M1 pairs (the four bytes of w) -> four f16x2, low nibble in the low half.
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// Two E4M3 pairs (the two halves of w) -> two f16x2.
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}

// 2^(e - 127) for byte `idx` of a word of E8M0 scales; e = 0 is the subnormal
// 2^-127 and e = 255 is +inf, as ldexp gives (src/core/numerics/quant.cpp:279-281).
__device__ __forceinline__ float e8m0_byte(uint32_t w, int idx) {
  const uint32_t e = __byte_perm(w, 0, 0x4440 + idx);
  return fmaxf(__uint_as_float(e << 23), __uint_as_float(0x00400000u));
}

// Thread-block cluster barrier (all threads of all CTAs of the cluster) and a
// load from the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Stages `nblk` activation blocks starting at block `first` of every row:
//   act: [k group of G elements][column][G halves], columns 2i (hi) and 2i+1 (lo)
//   cs : [block][kMaxCols] fp32, unit and unit / 2^11
// One warp per (row, block); lane l owns elements 4l..4l+3 and 128+4l..128+4l+3.
template <int G>
__device__ __forceinline__ void stage_f16(const F16Params& p, int first, int nblk, unsigned char* act,
                                          float* cs, int warp, int lane, int nwarps) {
  constexpr int kBatch = 4;
  const int items = p.m * nblk;
#pragma unroll 1
  for (int base = warp; base < items; base += nwarps * kBatch) {
    float4 x0[kBatch], x1[kBatch];
    int row[kBatch], blk[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int it = base + u * nwarps;
      row[u] = it / nblk;
      blk[u] = it - row[u] * nblk;
      x0[u] = x1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (it < items) {
        const float4* src = reinterpret_cast<const float4*>(p.a + static_cast<size_t>(row[u]) * p.k +
                                                            static_cast<size_t>(first + blk[u]) * kBlockElems);
        x0[u] = __ldg(src + lane);
        x1[u] = __ldg(src + 32 + lane);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (base + u * nwarps < items) {
        const float amax = fminf(
            __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(abs_max4(abs_max4(0.0f, x0[u]), x1[u])))),
            3.0e38f);
        const float unit = fmaxf(amax * (1.0f / 1024.0f), 1.0e-37f);
        const float c = __frcp_rn(unit);
        const int i = row[u], bl = blk[u];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float4 x = q == 0 ? x0[u] : x1[u];
          const float v0 = x.x * c, v1 = x.y * c, v2 = x.z * c, v3 = x.w * c;
          const uint32_t h01 = pack_half2(v0, v1), h23 = pack_half2(v2, v3);
          const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
          const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
          const uint32_t l01 = pack_half2((v0 - f01.x) * kLoScale, (v1 - f01.y) * kLoScale);
          const uint32_t l23 = pack_half2((v2 - f23.x) * kLoScale, (v3 - f23.y) * kLoScale);
          const int e = bl * kBlockElems + q * 128 + lane * 4;  // element inside the phase
          unsigned char* dst = act + (static_cast<size_t>(e / G) * p.ncols + 2 * i) * (2 * G) + (e % G) * 2;
          *reinterpret_cast<uint2*>(dst) = make_uint2(h01, h23);
          *reinterpret_cast<uint2*>(dst + 2 * G) = make_uint2(l01, l23);
        }
        if (lane < 2) cs[bl * kMaxCols + 2 * i + lane] = lane == 0 ? unit : unit * (1.0f / kLoScale);
      }
    }
  }
}

// SETS consumer warp sets (2, or 4 for launches with at most one CTA per SM: the sets split
// the chunks of k among them, which shortens every warp's chain of dependent chunks).
template <int FMT, int NCG, int SETS>
__global__ void __launch_bounds__((SETS * 4 + 1) * 32, SETS == 2 ? 2 : 1)
gemv_f16_staged_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                       const F16Params p) {
  constexpr int G = Fmt<FMT>::kGroup;
  constexpr int kChunkElems = Fmt<FMT>::kChunkElems;
  constexpr int kChunkBlocks = kChunkElems / kBlockElems;
  extern __shared__ unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: stages start on 1 KiB boundaries
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kConsumerWarps = SETS * p.rgs, kConsumerThreads = kConsumerWarps * 32;
  const int kTileRows = 16 * p.rgs, kStageBytes = p.rgs * kGroupStageBytes;
  const int kScaleBytes = FMT == kFmtMxfp4 ? p.rgs * kGroupScaleBytes : 0;
  // K split across the CTAs of a cluster: rank r takes chunks [r * cper, (r + 1) * cper)
  const int krank = p.ksplit > 1 ? static_cast<int>(blockIdx.x % p.ksplit) : 0;
  const int c_begin = krank * p.cper;
  const int nchunks_all = (p.nblocks + kChunkBlocks - 1) / kChunkBlocks;
  const int nchunks = max(0, min(p.cper, nchunks_all - c_begin));
  const int kb0 = c_begin * kChunkBlocks;  // first activation block of this CTA
  const int nblocks = max(0, min(p.nblocks - kb0, nchunks * kChunkBlocks));
  unsigned char* scales = smem + static_cast<size_t>(p.stages) * kStageBytes;
  unsigned char* act = scales + static_cast<size_t>(p.stages) * kScaleBytes;
  float* cs = reinterpret_cast<float*>(act + static_cast<size_t>(p.pblocks) * kBlockElems * p.ncols * 2);
  float* xchg = cs + static_cast<size_t>(p.pblocks) * kMaxCols;  // [SETS - 1][row groups][32 lanes][NCG*4]
  float* outbuf = xchg + (SETS - 1) * p.rgs * 32 * NCG * 4;       // [tile rows][NCG*8]
  uint64_t* full = reinterpret_cast<uint64_t*>(outbuf + kTileRows * NCG * 8);
  uint64_t* empty = full + p.stages;
  const unsigned char* zero_page = reinterpret_cast<const unsigned char*>(empty + p.stages);  // 16 zero bytes
  const int row0 = static_cast<int>(blockIdx.x / p.ksplit) * kTileRows;
  const bool producer = (tid == kConsumerThreads);

  if (tid < 4) reinterpret_cast<uint32_t*>(empty + p.stages)[tid] = 0u;
  if (producer) {
    tma_prefetch_descriptor(&wmap);
    if (FMT == kFmtMxfp4) tma_prefetch_descriptor(&smap);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], p.rgs);
    }
    mbar_fence_init();
  }
  __syncthreads();

  auto issue_chunk = [&](int c, int slot) {
    mbar_expect_tx(&full[slot], kStageBytes + kScaleBytes);
    // (128 bytes of a row, rows, 128-byte segments of the row): two segments per stage
    tma_load_3d(smem + static_cast<size_t>(slot) * kStageBytes, &wmap, 0, row0, 2 * (c_begin + c), &full[slot]);
    if (FMT == kFmtMxfp4)
      tma_load_2d(scales + static_cast<size_t>(slot) * kScaleBytes, &smap, 16 * (c_begin + c), row0, &full[slot]);
  };
  auto prologue = [&]() {
    if (producer) {
      const int first = nchunks < p.stages ? nchunks : p.stages;
      for (int c = 0; c < first; ++c) issue_chunk(c, c);
    }
  };
  if (p.pdl) {
    // Weights are not written by the kernel ahead of us (the launcher checked):
    // start their prefetch, then wait for that kernel's results to be visible.
    prologue();
    if (warp < kConsumerWarps && lane == 0 && warp < p.m)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.a + static_cast<size_t>(warp) * p.k));
    pdl_wait();
    pdl_trigger();
  }

  if (warp == kConsumerWarps) {
    if (!p.pdl) {
      // Touch one activation word first: the weight prefetch of all CTAs would
      // otherwise queue ahead of everybody's activation loads in the memory system.
      const float probe = __ldg(p.a + lane);
      if (probe != probe + 1.0f || lane >= 0) prologue();
    }
    if (lane == 0) {
      for (int c = p.stages; c < nchunks; ++c) {
        const RingUse use = ring_use(c, p.stages, SETS);
        const int s = use.slot;
        if (!mbar_wait(&empty[s], (use.round & 1) ^ 1, &g_f16_wait_timeouts)) break;
        issue_chunk(c, s);
      }
    }
    if (p.ksplit > 1) {  // the two cluster barriers of the epilogue
      cluster_sync();
      cluster_sync();
    }
    return;
  }

  const int gid = lane >> 2, tig = lane & 3;
  const int bx = warp / p.rgs, rg = warp - bx * p.rgs;  // warp set bx takes chunks c = bx (mod SETS)
  const int rowA = rg * 16 + gid;
  // Per-thread fragment addresses.  A lane whose column does not exist reads
  // the zero page with a zero stride, so the loop needs no predicates.
  const unsigned char* act_t[NCG];
  uint32_t act_grp[NCG];
#pragma unroll
  for (int g = 0; g < NCG; ++g) {
    const int col = g * 8 + gid;
    const bool valid = col < p.ncols;
    act_t[g] = valid ? act + col * (2 * G) + tig * (G / 2) : zero_page;  // G/4 halves per thread
    act_grp[g] = valid ? p.ncols * (2 * G) : 0;
  }
  const float* cs_t = cs + 2 * tig;  // this thread's two columns of a group
  // stage row r, 16-byte piece j: r * 128 + ((j ^ (r & 7)) << 4); r & 7 == gid for both MMA rows
  const uint32_t row_off = rowA * kSegBytes + tig * 4;
  const uint32_t seg_stride = kTileRows * kSegBytes;

  float o[NCG][4];
#pragma unroll
  for (int g = 0; g < NCG; ++g)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[g][e] = 0.0f;

  bool failed = false;
  int c = bx;
  // this set's ring slots bx, bx + SETS, ... in turn (see ring_use)
  const int owned = (p.stages - bx + SETS - 1) / SETS;
  int ring_idx = 0, ring_round = 0;
  for (int first = 0; first < nblocks; first += p.pblocks) {
    const int nblk = min(p.pblocks, nblocks - first);
    if (first > 0) asm volatile("bar.sync 1, %0;" ::"r"(kConsumerThreads) : "memory");
    stage_f16<G>(p, kb0 + first, nblk, act, cs, warp, lane, kConsumerWarps);
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerThreads) : "memory");
    const int chunk_end = (first + nblk + kChunkBlocks - 1) / kChunkBlocks;
    for (; c < chunk_end; c += SETS) {
      if (failed) continue;
      const int slot = bx + SETS * ring_idx;
      if (!mbar_wait(&full[slot], ring_round & 1, &g_f16_wait_timeouts)) {
        failed = true;
        continue;
      }
      const unsigned char* st = smem + static_cast<size_t>(slot) * kStageBytes + row_off;
      const int bl0 = c * kChunkBlocks - first;  // first block of the chunk inside the phase
      if (FMT == kFmtMxfp4) {
        const uint4 sA = *reinterpret_cast<const uint4*>(scales + static_cast<size_t>(slot) * kScaleBytes + rowA * 16);
        const uint4 sB = *reinterpret_cast<const uint4*>(scales + static_cast<size_t>(slot) * kScaleBytes + (rowA + 8) * 16);
        const uint32_t swA[4] = {sA.x, sA.y, sA.z, sA.w}, swB[4] = {sB.x, sB.y, sB.z, sB.w};
#pragma unroll
        for (int seg = 0; seg < 2; ++seg) {
          if (bl0 + seg >= nblk) break;  // a last chunk that holds one block only
          float t[NCG][4];
#pragma unroll
          for (int g = 0; g < NCG; ++g)
#pragma unroll
            for (int e = 0; e < 4; ++e) t[g][e] = 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // scale block 8 seg + j: one 16-byte piece of the row
            const unsigned char* pa = st + seg * seg_stride + ((j ^ gid) << 4);
            uint32_t ha[4], hb[4];
            cvt_e2m1x8(lds32(pa), ha);
            cvt_e2m1x8(lds32(pa + 8 * kSegBytes), hb);
            const float wa = e8m0_byte(swA[2 * seg + (j >> 2)], j & 3);
            const float wb = e8m0_byte(swB[2 * seg + (j >> 2)], j & 3);
#pragma unroll
            for (int g = 0; g < NCG; ++g) {
              const uint4 b = *reinterpret_cast<const uint4*>(act_t[g] + ((bl0 + seg) * 8 + j) * act_grp[g]);
              float part[4] = {0.f, 0.f, 0.f, 0.f};
              mma_f16_16816(part, ha[0], hb[0], ha[1], hb[1], b.x, b.y);
              mma_f16_16816(part, ha[2], hb[2], ha[3], hb[3], b.z, b.w);
              t[g][0] = fmaf(wa, part[0], t[g][0]);
              t[g][1] = fmaf(wa, part[1], t[g][1]);
              t[g][2] = fmaf(wb, part[2], t[g][2]);
              t[g][3] = fmaf(wb, part[3], t[g][3]);
            }
          }
#pragma unroll
          for (int g = 0; g < NCG; ++g) {
            const float2 c2 = *reinterpret_cast<const float2*>(cs_t + (bl0 + seg) * kMaxCols + g * 8);
            o[g][0] = fmaf(c2.x, t[g][0], o[g][0]);
            o[g][1] = fmaf(c2.y, t[g][1], o[g][1]);
            o[g][2] = fmaf(c2.x, t[g][2], o[g][2]);
            o[g][3] = fmaf(c2.y, t[g][3], o[g][3]);
          }
        }
      } else {
        float t[NCG][4];
#pragma unroll
        for (int g = 0; g < NCG; ++g)
#pragma unroll
          for (int e = 0; e < 4; ++e) t[g][e] = 0.0f;
#pragma unroll
        for (int seg = 0; seg < 2; ++seg) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // 16 elements: one MMA step
            const unsigned char* pa = st + seg * seg_stride + ((j ^ gid) << 4);
            uint32_t a0, a1, a2, a3;
            cvt_e4m3x4(lds32(pa), a0, a2);
            cvt_e4m3x4(lds32(pa + 8 * kSegBytes), a1, a3);
#pragma unroll
            for (int g = 0; g < NCG; ++g) {
              const uint2 b = *reinterpret_cast<const uint2*>(act_t[g] + (bl0 * 16 + seg * 8 + j) * act_grp[g]);
              mma_f16_16816(t[g], a0, a1, a2, a3, b.x, b.y);
            }
          }
        }
#pragma unroll
        for (int g = 0; g < NCG; ++g) {
          const float2 c2 = *reinterpret_cast<const float2*>(cs_t + bl0 * kMaxCols + g * 8);
          o[g][0] = fmaf(c2.x, t[g][0], o[g][0]);
          o[g][1] = fmaf(c2.y, t[g][1], o[g][1]);
          o[g][2] = fmaf(c2.x, t[g][2], o[g][2]);
          o[g][3] = fmaf(c2.y, t[g][3], o[g][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);
      if (++ring_idx == owned) {
        ring_idx = 0;
        ++ring_round;
      }
    }
  }

  // The two warps of a row group (even and odd chunks) add their partial sums; the
  // hi and lo columns of each activation row are then combined through shared memory.
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
  // With a K split the CTAs of the cluster hold partial sums of the same tile:
  // rank 0 adds them in rank order out of its peers' shared memory.
  if (p.ksplit > 1) cluster_sync();  // every CTA's outbuf is complete
  if (krank == 0) {
    for (int idx = tid; idx < p.m * kTileRows; idx += kConsumerThreads) {
      const int i = idx / kTileRows, rr = idx - i * kTileRows;
      if (row0 + rr < p.n) {
        const float* lo = outbuf + rr * (NCG * 8) + 2 * i + 1;
        float v = lo[0] + lo[-1];
        for (int r = 1; r < p.ksplit; ++r) v += ld_cluster_f32(lo, r) + ld_cluster_f32(lo - 1, r);
        if (FMT == kFmtFp8) v *= __ldg(p.row_scale + row0 + rr);
        p.c[static_cast<size_t>(i) * p.n + row0 + rr] = v;
      }
    }
  }
  if (p.ksplit > 1) cluster_sync();  // peers stay resident until they have been read
}

// ---- tensor-map cache
struct MapKey {
  const void* base;
  uint64_t n, k;
  int rgs, fmt;
  bool operator==(const MapKey& o) const {
    return base == o.base && n == o.n && k == o.k && rgs == o.rgs && fmt == o.fmt;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (k.n * 0x9E3779B97F4A7C15ull) ^ (k.k << 40) ^
           (static_cast<size_t>(k.rgs * 2 + k.fmt) << 58);
  }
};
struct MapPair {
  CUtensorMap weights, scales;
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, MapPair, MapKeyHash> g_maps;

int f16_tensor_maps(int fmt, const void* w, uint64_t n, uint64_t k, int rgs, MapPair* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{w, n, k, rgs, fmt};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return kOk;
  }
  const uint64_t row_bytes = fmt == kFmtMxfp4 ? k / 2 : k;
  MapPair pair{};
  // (128 bytes inside a row, rows, 128-byte segments of a row)
  const uint64_t dims[3] = {kSegBytes, n, row_bytes / kSegBytes};
  const uint64_t strides[2] = {row_bytes, kSegBytes};
  const uint32_t box[3] = {kSegBytes, static_cast<uint32_t>(16 * rgs), 2};
  int rc = encode_tensor_map(&pair.weights, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w, dims, strides, box, true);
  if (rc != kOk) return rc;
  if (fmt == kFmtMxfp4) {
    const uint64_t sdims[2] = {k / 32, n};
    const uint64_t sstrides[1] = {k / 32};
    const uint32_t sbox[2] = {16, static_cast<uint32_t>(16 * rgs)};
    rc = encode_tensor_map(&pair.scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                           static_cast<const unsigned char*>(w) + n * (k / 2), sdims, sstrides, sbox);
    if (rc != kOk) return rc;
  } else {
    pair.scales = pair.weights;
  }
  if (g_maps.size() > 65536) g_maps.clear();
  g_maps.emplace(key, pair);
  *out = pair;
  return kOk;
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}

// With `cost_only` the launch is planned but not issued, and its modelled time returned.
template <int FMT, int NCG, int SETS>
int launch_f16(const void* w, F16Params p, uint64_t n, uint64_t k, cudaStream_t st, double* cost_only) {
  constexpr int kChunkBlocks = Fmt<FMT>::kChunkElems / kBlockElems;
  const uint64_t nchunks_all = (static_cast<uint64_t>(p.nblocks) + kChunkBlocks - 1) / kChunkBlocks;
  const uint64_t per_block = static_cast<uint64_t>(kBlockElems) * p.ncols * 2;
  uint64_t max_blocks = (56u * 1024u) / per_block;
  max_blocks -= max_blocks % kChunkBlocks;
  if (max_blocks < 2u * kChunkBlocks) return kUnsupportedFeature;
  static const int regs = kernel_registers(gemv_f16_staged_kernel<FMT, NCG, SETS>);
  auto stage_bytes = [](int rgs) -> size_t {
    return static_cast<size_t>(rgs) * (kGroupStageBytes + (FMT == kFmtMxfp4 ? kGroupScaleBytes : 0));
  };
  // Activation phases of a CTA that owns `blocks` blocks: at most ~56 KiB of staged
  // activations at a time, phases of equal size, a whole number of chunks each.
  auto phase_blocks = [&](uint64_t blocks) -> uint64_t {
    const uint64_t phases = (blocks + max_blocks - 1) / max_blocks;
    uint64_t pblocks = (blocks + phases - 1) / phases;
    pblocks += (kChunkBlocks - pblocks % kChunkBlocks) % kChunkBlocks;
    return pblocks;
  };
  auto fixed_for = [&](uint64_t pblocks) {
    return [=](int rgs) -> size_t {
      return 1024 + pblocks * per_block + pblocks * kMaxCols * 4 + (SETS - 1) * rgs * 32 * NCG * 4 * 4 +
             16 * rgs * NCG * 8 * 4 + 2 * 8 * 16 + 128;
    };
  };
  // K split over a thread-block cluster (1, 2 or 4 CTAs per row tile): more CTAs
  // and shorter per-warp chains for shapes with few rows and a long k, at the
  // price of one exchange through distributed shared memory.  TSR_KSPLIT forces a factor.
  const int forced_split = env_int("TSR_KSPLIT", 0);
  StagedPlan plan{};
  uint64_t best_split = 0, best_cper = 0, best_pblocks = 0;
  double best_cost = 1e30;
  for (uint64_t ks = 1; ks <= 4; ks *= 2) {
    if (forced_split > 0 && static_cast<uint64_t>(forced_split) != ks) continue;
    const uint64_t cper = (nchunks_all + ks - 1) / ks;
    if (ks > 1 && (cper < 2 || cper * (ks - 1) >= nchunks_all)) continue;  // every rank has work
    const uint64_t pblocks = phase_blocks(cper * kChunkBlocks);
    StagedPlan cand{};
    if (!plan_staged(n, ks, cper * kChunkBlocks, cper, 12, regs, fixed_for(pblocks), stage_bytes, &cand, SETS)) continue;
    // measured: a cluster launch with its two cluster barriers costs about 5 us
    // (2 CTAs) to 8 us (4 CTAs) over the plain one, so only a long k pays for it
    const double cost = cand.cost + (ks == 1 ? 0.0 : ks == 2 ? 5.0 : 8.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      plan = cand;
      best_split = ks;
      best_cper = cper;
      best_pblocks = pblocks;
    }
  }
  if (best_split == 0) return kUnsupportedFeature;
  if (cost_only != nullptr) {
    *cost_only = best_cost;
    return kOk;
  }
  auto fixed = fixed_for(best_pblocks);
  const int forced_rgs = env_int("TSR_RGS", 0);
  if (forced_rgs >= 1 && forced_rgs <= 4) {
    plan.rgs = forced_rgs;
    plan.smem = fixed(forced_rgs) + plan.stages * stage_bytes(forced_rgs);
  }
  const int forced = env_int("TSR_STAGES", 0);
  if (forced >= SETS && forced <= 16 &&
      fixed(plan.rgs) + forced * stage_bytes(plan.rgs) <= static_cast<size_t>(kMaxSmem)) {
    plan.stages = forced;
    plan.smem = fixed(plan.rgs) + forced * stage_bytes(plan.rgs);
  }
  if (plan.smem > static_cast<size_t>(kMaxSmem)) return kUnsupportedFeature;
  p.pblocks = static_cast<int>(best_pblocks);
  p.rgs = plan.rgs;
  p.stages = plan.stages;
  p.ksplit = static_cast<int>(best_split);
  p.cper = static_cast<int>(best_cper);
  MapPair maps;
  if (int rc = f16_tensor_maps(FMT, w, n, k, plan.rgs, &maps)) return rc;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&gemv_f16_staged_kernel<FMT, NCG, SETS>), kMaxSmem)) return rc;
  const uint64_t th = 16u * plan.rgs;
  const dim3 grid(static_cast<unsigned>(((n + th - 1) / th) * best_split));
  const size_t w_bytes = FMT == kFmtMxfp4 ? n * (k / 2) + n * (k / 32) : n * k;
  p.pdl = pdl_allowed(st, w, w_bytes, p.c, static_cast<size_t>(p.m) * n * 4) ? 1 : 0;
  if (env_int("TSR_PLAN_DEBUG", 0))
    std::fprintf(stderr, "f16 plan fmt=%d sets=%d m=%d n=%llu k=%llu: ksplit=%llu cper=%llu pblocks=%llu rgs=%d stages=%d smem=%zu grid=%u cost=%.2f\n",
                 FMT, SETS, p.m, (unsigned long long)n, (unsigned long long)k, (unsigned long long)best_split,
                 (unsigned long long)best_cper, (unsigned long long)best_pblocks, plan.rgs, plan.stages, plan.smem,
                 grid.x, best_cost);
  launch_kernel_cluster(gemv_f16_staged_kernel<FMT, NCG, SETS>, grid, dim3((SETS * plan.rgs + 1) * 32), plan.smem, st,
                        p.pdl != 0, static_cast<unsigned>(best_split), maps.weights, maps.scales, p);
  return check_launch();
}

template <int FMT>
int staged_f16(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n,
               uint64_t k, cudaStream_t st) {
  // whole chunks only; 16-byte aligned rows and scale rows
  if (m > 8 || k % Fmt<FMT>::kChunkElems != 0 || (reinterpret_cast<uintptr_t>(w) & 15u) ||
      env_int("TSR_DISABLE_STAGED", 0))
    return kUnsupportedFeature;
  F16Params p{a, c, scale, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
              static_cast<int>(k / kBlockElems), 0, 0, static_cast<int>(2 * m), 0, 4, 1, 0};
  // two consumer sets, or four when the model says the warps' own chains of chunks
  // (not the SM's throughput) set the time: few CTAs, long k
  auto run = [&](auto ncg) -> int {
    constexpr int kNcg = decltype(ncg)::value;
    double c2 = 0.0, c4 = 0.0;
    const int r2 = launch_f16<FMT, kNcg, 2>(w, p, n, k, st, &c2);
    const int r4 = launch_f16<FMT, kNcg, 4>(w, p, n, k, st, &c4);
    const int forced_sets = env_int("TSR_SETS", 0);
    const bool four = forced_sets == 4 ? r4 == kOk : forced_sets == 2 ? r2 != kOk && r4 == kOk
                                                                      : r4 == kOk && (r2 != kOk || (four_sets_worthwhile(n, 1) && c4 + 0.3 < c2));
    if (four) return launch_f16<FMT, kNcg, 4>(w, p, n, k, st, nullptr);
    if (r2 != kOk) return r2;
    return launch_f16<FMT, kNcg, 2>(w, p, n, k, st, nullptr);
  };
  if (m <= 4) return run(std::integral_constant<int, 1>{});
  return run(std::integral_constant<int, 2>{});
}

}  // namespace

// Return kUnsupportedFeature when the shape is outside what the staged kernel
// covers; the caller then uses the general warp-per-row family.
int staged_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                      cudaStream_t st) {
  return staged_f16<kFmtMxfp4>(a, w, nullptr, c, m, n, k, st);
}

int staged_gemm_fp8(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n,
                    uint64_t k, cudaStream_t st) {
  return staged_f16<kFmtFp8>(a, w, scale, c, m, n, k, st);
}

int staged_f16_set_error_word(unsigned int* word) { return set_host_error_word(word); }

int staged_f16_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_f16_wait_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}

}  // namespace tsr
