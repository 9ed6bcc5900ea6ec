// Pieces shared by the staged tensor-pipe GEMV kernels (Q4_K: gemv_mma.cu,
// Q6_K: gemv_q6k_mma.cu, MXFP4/FP8: gemv_f16_mma.cu): launch parameters,
// shared-memory loads, the int8 digit expansion of the activations and its
// staging into shared memory (the two K-quant kernels), and the host-side
// launch plan (tile height, CTAs per SM, ring depth) that all three use.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "codec.cuh"
#include "launch.h"
#include "pipeline.cuh"
#include "tp_device.cuh"

namespace tsr {
namespace staged {

constexpr int kStagedConsumerWarps = 8;                         // two sets of four row groups
constexpr int kStagedThreads = kStagedConsumerWarps * 32 + 32;  // plus the producer warp
constexpr int kMaxSmem = 227 * 1024;
constexpr int kMaxCols = 16;

// One weight tensor of a launch.  All targets of a launch share the activations,
// m, k, the split and the tile height; the launch's tile list is the
// concatenation of the targets' row tiles.
struct StagedTarget {
  float* c;        // [m][n] outputs (or `split` such regions when the split is left to the caller)
  int n;           // weight rows
  int tile_begin;  // index of this target's first tile in the launch's tile list
  int aux;         // format specific (Q6_K: byte shift of the odd-row tensor map)
  // residual add folded into the output: add_out[e] = add_src[e] + C[e] is written besides C
  // (null: none).  add_out may be add_src or c itself, not a shifted overlap of either.
  const float* add_src;
  float* add_out;
};

enum : int {
  kSplitCaller = 0,    // chunk y of k goes to region y of each target (stride m*n): the caller adds them
  kSplitInLaunch = 1,  // the last CTA of a tile to finish adds the chunks in chunk order
  // The CTAs (x, 0..split-1) form a thread-block cluster: chunks 1.. store their sums into the
  // shared memory of chunk 0's CTA and signal an mbarrier there; that CTA adds them in chunk
  // order.  A CTA works through at most kClusterTiles tiles (one receive buffer per tile).
  kSplitCluster = 2,
};
// What a kernel variant does after a tile's sums (template parameter OUT of the staged kernels).
enum : int { kOutGeneral = 0, kOutPlain = 1, kOutRanks = 2 };
constexpr int kClusterTiles = 2;
// The cluster form is compiled only with -DTSR_CLUSTER_SPLIT=1 (experiments).
#ifndef TSR_CLUSTER_SPLIT
#define TSR_CLUSTER_SPLIT 0
#endif

struct StagedParams {
  const float* a;
  int m, k;
  int per;     // blocks per split chunk
  int stages;  // ring depth
  int terms;   // int8 digits per activation row
  int ncols;   // m * terms
  int debug;   // experiment switches: 1 skips activation staging, 2 skips the block math
  int pdl;     // launched as a programmatic dependent: prefetch weights, then wait for the stream
  int rgs;     // 16-row groups per CTA (1..4): the tile has 16*rgs rows
  int sets;    // consumer warp sets (2 or 4): sets*rgs consumer warps; set s takes the chunks c = s (mod sets)
  int ntargets, total_tiles;
  int split_mode;
  StagedTarget tgt[kMaxGroup];
  // kSplitInLaunch: partial tiles [chunk][tile][m][tile rows] and one arrival count per tile (zero at rest)
  float* part;
  unsigned int* tickets;
  TpTail tp;  // sum over tensor-parallel ranks after the local sum (world 1: none)
  // What is done to the activations on their way into shared memory (kProNone: nothing).
  //   kProSiluMul: a holds the gate, a2 the up vector, the projection reads silu(a) * a2
  //                (SiluMulRef, src/core/numerics/norm.cpp:211-225 of the reference)
  //   kProRmsNorm: a2 holds the k norm weights, the projection reads a / sqrt(mean(a^2) + eps) * a2
  //                row by row (RmsNormRef, src/core/numerics/norm.cpp:7-32)
  //   kProRmsNormLate: the same where every CTA stages whole rows (k not split): a * a2 is
  //                staged, the squares are added up on the way, and the row's gain multiplies the
  //                sums in the output stage (it is a factor of the whole row); a_out is written at
  //                the end of the kernel, every CTA a share
  // a_out (may be null) receives those activations, [m][k] like a, written by the CTAs of
  // tile column 0; it must not overlap a or a2.
  int pro;
  float eps;
  const float* a2;
  float* a_out;
  // a holds bf16 values ([m][k], 2 bytes each) / the targets' c are bf16 storage ([m][n], 2 bytes
  // each; the sums are rounded to nearest even).  The partial sums and the exchange between
  // ranks stay fp32.
  int a_bf16, c_bf16;
};

// Rounds to bf16 like RoundBf16Ref (src/core/numerics/quant.cpp:231-243 of the reference).
__device__ __forceinline__ unsigned short bf16_bits_rn(float v) {
  unsigned int u = __float_as_uint(v);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<unsigned short>(u >> 16);
}
__device__ __forceinline__ void store_output(const StagedParams& p, float* c, size_t e, float v) {
  if (p.c_bf16)
    reinterpret_cast<unsigned short*>(c)[e] = bf16_bits_rn(v);
  else
    c[e] = v;
}
__device__ __forceinline__ float4 bf16x4_to_float4(uint2 b) {
  return make_float4(__uint_as_float(b.x << 16), __uint_as_float(b.x & 0xFFFF0000u), __uint_as_float(b.y << 16),
                     __uint_as_float(b.y & 0xFFFF0000u));
}

// Which target a tile of the launch's tile list belongs to, and that target by value.
// The kernel parameters are read with constant indices only (a run-time index into a
// parameter array would make the compiler keep the whole array in registers or copy it
// to local memory), hence the unrolled compares.
__device__ __forceinline__ int target_of_tile(const StagedParams& p, int tile) {
  int g = 0;
#pragma unroll
  for (int i = 1; i < kMaxGroup; ++i)
    if (i < p.ntargets && tile >= p.tgt[i].tile_begin) g = i;
  return g;
}
__device__ __forceinline__ StagedTarget target_by_index(const StagedParams& p, int g) {
  StagedTarget t = p.tgt[0];
#pragma unroll
  for (int i = 1; i < kMaxGroup; ++i)
    if (g == i) t = p.tgt[i];
  return t;
}
// Address of element g of an array of kMaxGroup tensor maps in the kernel parameters.
__device__ __forceinline__ const CUtensorMap* map_by_index(const CUtensorMap* maps, int g) {
  const CUtensorMap* m = &maps[0];
#pragma unroll
  for (int i = 1; i < kMaxGroup; ++i)
    if (g == i) m = &maps[i];
  return m;
}

__device__ __forceinline__ uint4 lds128(const unsigned char* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ uint2 lds64(const unsigned char* p) {
  return *reinterpret_cast<const uint2*>(p);
}

// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col), zero accumulate input
__device__ __forceinline__ void mma_u8s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Quantise four activations to signed base-256 digits.  With c = 2^shift / s
// the value X = rint(x * c) fits 23 bits, so t = x*c + 1.5*2^23 holds X in its
// low mantissa bits; adding 0x8080 and flipping those two bits turns the three
// low bytes of the word into balanced digits (X = q1*65536 + q2*256 + q3 with
// q2, q3 in [-128,127]).  No conversion instruction and no clamp is needed.
// Three digits use shift 15 (|X| <= 127*2^15 < 2^22), two digits shift 7.
// w[0] is the most significant digit of the four values, packed one per byte.
__device__ __forceinline__ void quantise4(float4 x, float c, int terms, uint32_t (&w)[3]) {
  constexpr float kMagic = 12582912.0f;                        // 1.5 * 2^23
  constexpr uint32_t kBias = 0x8080u - 0x4B400000u;            // remove the magic, add the digit bias
  const uint32_t y0 = (__float_as_uint(fmaf(x.x, c, kMagic)) + kBias) ^ 0x8080u;
  const uint32_t y1 = (__float_as_uint(fmaf(x.y, c, kMagic)) + kBias) ^ 0x8080u;
  const uint32_t y2 = (__float_as_uint(fmaf(x.z, c, kMagic)) + kBias) ^ 0x8080u;
  const uint32_t y3 = (__float_as_uint(fmaf(x.w, c, kMagic)) + kBias) ^ 0x8080u;
  // byte j of every word -> one word per digit
  const uint32_t lo01 = __byte_perm(y0, y1, 0x5140), lo23 = __byte_perm(y2, y3, 0x5140);  // bytes 0,1 of each
  const uint32_t b2 = __byte_perm(__byte_perm(y0, y1, 0x0062), __byte_perm(y2, y3, 0x0062), 0x5410);
  const uint32_t b1 = __byte_perm(lo01, lo23, 0x7632);
  const uint32_t b0 = __byte_perm(lo01, lo23, 0x5410);
  if (terms == 3) {
    w[0] = b2;
    w[1] = b1;
    w[2] = b0;
  } else {
    w[0] = b1;
    w[1] = b0;
    w[2] = 0;
  }
}

__device__ __forceinline__ float abs_max4(float m, float4 x) {
  return fmaxf(m, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
}

// Activation staging.  Layout in shared memory:
//   act : [block][sub-block 0..7][column][32 bytes]   int8 digits in k order
//   sums: [block][digit plane 0..1][column][GROUPS bytes]  digit sums of every
//         256/GROUPS-element group (GROUPS = 8: Q4_K sub-blocks, 16: Q6_K
//         scale groups), S = D0 + 128*D1 with D0 in [-64,63]
//   cs  : [block][kMaxCols] fp32                       column scale s_block * 256^-digit
// Every 256-element block of an activation row has its own scale (its
// largest magnitude / 127), so one warp stages a block on its own: lane l
// owns elements 4l..4l+3 and 128+4l..128+4l+3, the block maximum is one warp
// reduction, and no CTA-wide pass is needed.  A warp works on kStageBatch
// blocks at a time so that their dependent chains overlap.
#ifndef TSR_STAGE_BATCH
#define TSR_STAGE_BATCH 4
#endif
constexpr int kStageBatch = TSR_STAGE_BATCH;

// Phase 1 of a block: scale, digits, column scales.
__device__ __forceinline__ void stage_digits(const StagedParams& p, int i, int bl, float4 x0, float4 x1,
                                             unsigned char* act, float* cs, int lane) {
  // non-negative floats order like their bit patterns
  const float amax = fminf(
      __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(abs_max4(abs_max4(0.0f, x0), x1)))),
      3.0e38f);
  // x ~= unit * X with X = rint(x / unit), |X| <= 127 * 2^shift.  The floor on
  // the unit keeps its reciprocal finite for all-zero and denormal-sized blocks.
  const float inv_top = p.terms == 3 ? (1.0f / (127.0f * 32768.0f)) : (1.0f / (127.0f * 128.0f));
  const float unit = fmaxf(amax * inv_top, 1.0e-37f);
  const float c = __frcp_rn(unit);
  uint32_t w0[3], w1[3];
  quantise4(x0, c, p.terms, w0);
  quantise4(x1, c, p.terms, w1);
  // lane l: elements 4l.. -> sub-block l/8; elements 128+4l.. -> sub-block 4 + l/8
  const int sb = lane >> 3, in_sb = (lane & 7) * 4;
  unsigned char* dst0 = act + ((bl * 8 + sb) * p.ncols + i * p.terms) * 32 + in_sb;
  unsigned char* dst1 = dst0 + 4 * p.ncols * 32;
  *reinterpret_cast<uint32_t*>(dst0) = w0[0];
  *reinterpret_cast<uint32_t*>(dst1) = w1[0];
  *reinterpret_cast<uint32_t*>(dst0 + 32) = w0[1];
  *reinterpret_cast<uint32_t*>(dst1 + 32) = w1[1];
  if (p.terms == 3) {
    *reinterpret_cast<uint32_t*>(dst0 + 64) = w0[2];
    *reinterpret_cast<uint32_t*>(dst1 + 64) = w1[2];
  }
  if (lane < p.terms) {
    // digit `lane` (most significant first) weighs 256^(terms-1-lane) units
    const float weight = unit * (lane == p.terms - 1 ? 1.0f : lane == p.terms - 2 ? 256.0f : 65536.0f);
    cs[bl * kMaxCols + i * p.terms + lane] = weight;
  }
}

// Phase 2 of a block, after the warp's digit stores are visible: lane
// (digit t, sub-block g) of the first 8 * terms lanes sums the 32 digits of
// its sub-block (two halves for GROUPS = 16) and stores them as two planes.
template <int GROUPS>
__device__ __forceinline__ void stage_sums(const StagedParams& p, int i, int bl, const unsigned char* act,
                                           unsigned char* sums, int lane) {
  const int t = lane >> 3, g = lane & 7;
  if (t >= p.terms) return;
  const int col = i * p.terms + t;
  const uint4* src = reinterpret_cast<const uint4*>(act + ((bl * 8 + g) * p.ncols + col) * 32);
  const uint4 u = src[0], v = src[1];
  const int lo = __dp4a(static_cast<int>(u.x), 0x01010101, __dp4a(static_cast<int>(u.y), 0x01010101, 0)) +
                 __dp4a(static_cast<int>(u.z), 0x01010101, __dp4a(static_cast<int>(u.w), 0x01010101, 0));
  const int hi = __dp4a(static_cast<int>(v.x), 0x01010101, __dp4a(static_cast<int>(v.y), 0x01010101, 0)) +
                 __dp4a(static_cast<int>(v.z), 0x01010101, __dp4a(static_cast<int>(v.w), 0x01010101, 0));
  unsigned char* sp = sums + ((bl * 2) * p.ncols + col) * GROUPS;
  const int plane = p.ncols * GROUPS;
  if (GROUPS == 8) {
    const int a = lo + hi, h = (a + 64) >> 7;
    sp[g] = static_cast<unsigned char>(a - 128 * h);
    sp[plane + g] = static_cast<unsigned char>(h);
  } else {
    const int h0 = (lo + 64) >> 7, h1 = (hi + 64) >> 7;
    const unsigned int d0 = ((lo - 128 * h0) & 0xFF) | (((hi - 128 * h1) & 0xFF) << 8);
    const unsigned int d1 = (h0 & 0xFF) | ((h1 & 0xFF) << 8);
    *reinterpret_cast<unsigned short*>(sp + 2 * g) = static_cast<unsigned short>(d0);
    *reinterpret_cast<unsigned short*>(sp + plane + 2 * g) = static_cast<unsigned short>(d1);
  }
}

// Stages the activation blocks [k0, k0 + per*256) of all m rows.  A kernel
// launched as a programmatic dependent (p.pdl) waits for the stream in here,
// before its first activation load; every thread of the CTA reaches that wait.
// The kernels let their own dependents go late, when a CTA has consumed the last
// chunk of its last tile: measured on a decode step of mixed launches, letting
// them go right after the wait (so that the next launch's CTAs sit resident,
// their first weights fetched, for the whole main loop) cost 11 % of the step.
__device__ __forceinline__ float4 silu_mul4(float4 g, float4 u) {
  return make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y,
                     g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
}
__device__ __forceinline__ float4 scale4(float4 x, float gain, float4 w) {
  return make_float4(x.x * gain * w.x, x.y * gain * w.y, x.z * gain * w.z, x.w * gain * w.w);
}

// `scratch`: (consumer warps + 1) * m floats of shared memory that nothing else uses
// during the staging (only touched for kProRmsNorm).
// PRO = false compiles the elementwise steps and the bf16 input out (p.pro and p.a_bf16 must
// then be zero): the staging code is what every launch runs before its first weight, and the
// smaller form made the 27B-class step 3.8 % faster.
template <int GROUPS, bool PRO, typename AfterFirstLoads>
__device__ __forceinline__ void stage_activations(const StagedParams& p, int k0, unsigned char* act,
                                                  unsigned char* sums, float* cs, float* scratch,
                                                  AfterFirstLoads after_first_loads) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // The producer warp only issues the weight copies: its first TMA instruction
  // can wait on the descriptor fetch, which must not hold up a share of the staging.
  const int kWarps = p.sets * p.rgs;
  if (warp >= kWarps) {
    if (p.pdl) {
      pdl_wait();
      return;
    }
    // Touch one activation word first: the weight prefetch of all CTAs would
    // otherwise queue ahead of everybody's activation loads in the memory system.
    const float probe = __ldg(p.a + ((k0 < p.k ? k0 : 0) >> p.a_bf16) + lane);  // bf16: half the bytes per element
    if (probe != probe + 1.0f || lane >= 0) after_first_loads();
    return;
  }
  const int items = p.m * p.per;  // (activation row, block) pairs, row-major
  if (p.pdl) {
    // Translate the activation pages while waiting (a prefetch reads no data into this SM).
    if (lane == 0 && warp < items)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(
          p.a + ((static_cast<size_t>(warp / p.per) * p.k + k0 + (warp % p.per) * kBlockElems) >> p.a_bf16)));
    pdl_wait();
  }
  const float* gain = scratch + kWarps * p.m;
  if (PRO && p.pro == kProRmsNorm) {
    // Every CTA needs the mean square of whole rows: each warp sums a share, the shares are
    // added in warp order.
    const int nthreads = kWarps * 32;
#pragma unroll 1
    for (int i = 0; i < p.m; ++i) {
      const float4* row = reinterpret_cast<const float4*>(p.a + static_cast<size_t>(i) * p.k);
      float s = 0.0f;
      for (int q = threadIdx.x; q < p.k / 4; q += nthreads) {
        const float4 v = __ldg(row + q);
        s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s))));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
      if (lane == 0) scratch[i * kWarps + warp] = s;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    if (threadIdx.x < p.m) {
      float s = 0.0f;
      for (int w = 0; w < kWarps; ++w) s += scratch[threadIdx.x * kWarps + w];
      scratch[kWarps * p.m + threadIdx.x] = 1.0f / sqrtf(s / static_cast<float>(p.k) + p.eps);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
  }
  const bool writes_out = PRO && p.a_out != nullptr && blockIdx.x == 0;
#pragma unroll 1
  for (int base = warp; base < items; base += kWarps * kStageBatch) {
    float4 x0[kStageBatch], x1[kStageBatch];
    float4 w0[kStageBatch], w1[kStageBatch];  // kProRmsNormLate only
    int row[kStageBatch], blk[kStageBatch];
#pragma unroll
    for (int u = 0; u < kStageBatch; ++u) {
      const int it = base + u * kWarps;
      row[u] = it / p.per;
      blk[u] = it - row[u] * p.per;
      x0[u] = x1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (it < items && k0 + blk[u] * kBlockElems < p.k) {
        const size_t first = static_cast<size_t>(row[u]) * p.k + k0 + blk[u] * kBlockElems;
        if (PRO && p.a_bf16) {
          const uint2* src = reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(p.a) + first);
          x0[u] = bf16x4_to_float4(__ldg(src + lane));
          x1[u] = bf16x4_to_float4(__ldg(src + 32 + lane));
        } else {
          const float4* src = reinterpret_cast<const float4*>(p.a + first);
          x0[u] = __ldg(src + lane);
          x1[u] = __ldg(src + 32 + lane);
        }
        if (PRO && p.pro == kProRmsNormLate) {
          // the norm weights of the block; squares and products follow once every load is out
          const float4* nw = reinterpret_cast<const float4*>(p.a2 + k0 + blk[u] * kBlockElems);
          w0[u] = __ldg(nw + lane);
          w1[u] = __ldg(nw + 32 + lane);
        } else if (PRO && p.pro != kProNone) {
          const size_t at = static_cast<size_t>(row[u]) * p.k + k0 + blk[u] * kBlockElems;
          if (p.pro == kProSiluMul) {
            const float4* up = reinterpret_cast<const float4*>(p.a2 + at);
            x0[u] = silu_mul4(x0[u], __ldg(up + lane));
            x1[u] = silu_mul4(x1[u], __ldg(up + 32 + lane));
          } else {
            const float4* nw = reinterpret_cast<const float4*>(p.a2 + k0 + blk[u] * kBlockElems);
            x0[u] = scale4(x0[u], gain[row[u]], __ldg(nw + lane));
            x1[u] = scale4(x1[u], gain[row[u]], __ldg(nw + 32 + lane));
          }
          if (writes_out) {
            float4* dst = reinterpret_cast<float4*>(p.a_out + at);
            dst[lane] = x0[u];
            dst[32 + lane] = x1[u];
          }
        }
      }
    }
    if (PRO && p.pro == kProRmsNormLate) {
#pragma unroll
      for (int u = 0; u < kStageBatch; ++u) {
        const int it = base + u * kWarps;
        if (it < items) {
          // squares of this lane's eight values; the warp's total goes to scratch[item]
          float ss = 0.0f;
          ss = fmaf(x0[u].x, x0[u].x, fmaf(x0[u].y, x0[u].y, fmaf(x0[u].z, x0[u].z, fmaf(x0[u].w, x0[u].w, ss))));
          ss = fmaf(x1[u].x, x1[u].x, fmaf(x1[u].y, x1[u].y, fmaf(x1[u].z, x1[u].z, fmaf(x1[u].w, x1[u].w, ss))));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
          if (lane == 0) scratch[it] = ss;
          x0[u] = scale4(x0[u], 1.0f, w0[u]);
          x1[u] = scale4(x1[u], 1.0f, w1[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kStageBatch; ++u)
      if (base + u * kWarps < items) stage_digits(p, row[u], blk[u], x0[u], x1[u], act, cs, lane);
    __syncwarp();
#pragma unroll
    for (int u = 0; u < kStageBatch; ++u)
      if (base + u * kWarps < items) stage_sums<GROUPS>(p, row[u], blk[u], act, sums, lane);
  }
}

// kProRmsNormLate, after the staging and a CTA-wide barrier: consumer thread i < m adds the
// squares of row i (block order) and stores the row's gain; the consumer threads then meet on
// barrier 1 (the scratch area is reused by the first tile's output stage).
__device__ __forceinline__ void rms_late_gain(const StagedParams& p, const float* scratch, float* gain, int tid,
                                              int nthreads) {
  if (tid < p.m) {
    float s = 0.0f;
    for (int b = 0; b < p.per; ++b) s += scratch[tid * p.per + b];
    gain[tid] = 1.0f / sqrtf(s / static_cast<float>(p.k) + p.eps);
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
// kProRmsNormLate, at the end of the kernel: a_out = a * gain * a2 (the rmsnorm's own output
// buffer) is written by the CTAs that had a tile less than the others (they would idle
// otherwise), or by all CTAs, a share each, when every CTA had the same number of tiles.
__device__ __forceinline__ void rms_late_write(const StagedParams& p, const float* gain, int cta, int ctas, int tid,
                                               int nthreads) {
  if (p.a_out == nullptr) return;
  const int with_more = p.total_tiles % ctas;  // CTAs 0 .. with_more-1 have one tile more
  int writers = ctas, me = cta;
  if (with_more != 0) {
    writers = ctas - with_more;
    me = cta - with_more;
    if (me < 0) return;
  }
  const int per_row = p.k / 4, total = p.m * per_row;
  const int share = (total + writers - 1) / writers;
  const int end = min(total, (me + 1) * share);
  for (int q = me * share + tid; q < end; q += nthreads) {
    const int i = q / per_row, c4 = q - i * per_row;
    const float4 x = __ldg(reinterpret_cast<const float4*>(p.a) + q);
    const float4 w = __ldg(reinterpret_cast<const float4*>(p.a2) + c4);
    reinterpret_cast<float4*>(p.a_out)[q] = scale4(x, gain[i], w);
  }
}

// What the consumer threads of a CTA do once a tile's sums sit in shared memory
// (`value(i, rr)` returns the sum of activation row i and tile row rr): write
// them out, or first add the split chunks of k (kSplitInLaunch) and then the
// tensor-parallel ranks.  Every consumer thread of the CTA calls this with the
// same arguments; it synchronises them on named barrier 1.  s_flag is one word
// of shared memory.  Returns nothing; a CTA that was not the last of its tile
// simply leaves without writing outputs.
template <typename ValueFn>
__device__ __forceinline__ void finish_tile(const StagedParams& p, const StagedTarget& tg, int tile, int row0,
                                            int tile_rows, int chunk_y, int nsplit, unsigned int epoch, int tid,
                                            int nthreads, unsigned int* s_flag, int it, uint64_t* recv_bar,
                                            float* recv, unsigned int* timeouts, ValueFn value) {
  // nthreads is a multiple of tile_rows (two or four warps per 16 rows): a thread keeps one
  // tile row rr and takes the activation rows i0, i0 + per_pass, ...
  const int per_pass = nthreads / tile_rows;
  const int i0 = tid / tile_rows, rr = tid - i0 * tile_rows;
  const bool row_ok = row0 + rr < tg.n;
  const size_t col = static_cast<size_t>(row0 + rr);
  if (p.split_mode == kSplitCaller) {
    float* cout = tg.c + static_cast<size_t>(chunk_y) * p.m * tg.n + col;
#pragma unroll 1
    for (int i = i0; i < p.m; i += per_pass)
      if (row_ok) cout[static_cast<size_t>(i) * tg.n] = value(i, rr);
    return;
  }
  const size_t tile_floats = static_cast<size_t>(p.m) * tile_rows;
#if TSR_CLUSTER_SPLIT
  const bool clustered = p.split_mode == kSplitCluster && nsplit > 1;
#else
  constexpr bool clustered = false;
#endif
  const float* received = recv + static_cast<size_t>(it) * (nsplit - 1) * tile_floats + rr;  // tile `it` of this CTA
#if TSR_CLUSTER_SPLIT
  if (clustered) {
    if (chunk_y != 0) {
      const uint32_t remote =
          cluster_map(smem_u32(recv + (static_cast<size_t>(it) * (nsplit - 1) + (chunk_y - 1)) * tile_floats + rr), 0);
#pragma unroll 1
      for (int i = i0; i < p.m; i += per_pass) st_cluster_f32(remote + i * tile_rows * 4, value(i, rr));
      // the barrier orders the CTA's stores before thread 0's arrival, whose release (cluster
      // scope) and the receiver's acquire order them before the receiver's loads
      asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
      if (tid == 0) mbar_arrive_remote(cluster_map(smem_u32(recv_bar + it), 0));
      return;
    }
    mbar_wait_cluster(recv_bar + it, 0, timeouts);  // bounded; on a timeout the sums below are wrong and the host is told
  } else
#endif
  if (nsplit > 1) {
    float* mine = p.part + (static_cast<size_t>(chunk_y) * p.total_tiles + tile) * tile_floats + rr;
#pragma unroll 1
    for (int i = i0; i < p.m; i += per_pass) __stcg(mine + i * tile_rows, value(i, rr));
    // The CTA's stores are ordered before the ticket by the barrier (CTA scope) and the
    // ticket's release (GPU scope); the last CTA's acquire on the ticket and its barrier
    // order the other chunks' stores before the loads below.  No thread needs a full fence.
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    if (tid == 0) {
      unsigned int t;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(p.tickets + tile) : "memory");
      *s_flag = (t == static_cast<unsigned int>(nsplit - 1)) ? 1u : 0u;
      if (*s_flag) p.tickets[tile] = 0u;  // every chunk has arrived: ready for the next launch
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    if (*s_flag == 0u) return;
  }
  const bool tp = p.tp.world > 1;
  // with ranks: every thread sends its own values to all ranks, then waits for the same
  // elements of all ranks in its own slots: no barrier, no flag (tp_device.cuh)
  const size_t mine_off = tp ? tp_slot_offset(p.tp, epoch, p.tp.rank) : 0;
  const float* parts = p.part + static_cast<size_t>(tile) * tile_floats + rr;
#pragma unroll 1
  for (int i = i0; i < p.m; i += per_pass) {
    float v;
    if (clustered) {
      v = value(i, rr);  // chunk 0, then the others in chunk order
#pragma unroll 1
      for (int y = 1; y < nsplit; ++y) v += received[(y - 1) * tile_floats + i * tile_rows];
    } else if (nsplit > 1) {
      // chunk order, starting from zero: the order of the reference's gemm_vec_reduce
      v = 0.0f;
#pragma unroll 1
      for (int y = 0; y < nsplit; ++y) v += __ldcg(parts + static_cast<size_t>(y) * p.total_tiles * tile_floats + i * tile_rows);
    } else {
      v = value(i, rr);
    }
    if (!row_ok) continue;
    const size_t e = static_cast<size_t>(i) * tg.n + col;
    if (tp) {
      tp_push(p.tp, mine_off + e, v);
    } else {
      store_output(p, tg.c, e, v);
      if (tg.add_out != nullptr) tg.add_out[e] = tg.add_src[e] + v;
    }
  }
  if (!tp || !row_ok) return;
#pragma unroll 1
  for (int i = i0; i < p.m; i += per_pass) {
    const size_t e = static_cast<size_t>(i) * tg.n + col;
    const float v = tp_wait_sum(p.tp, epoch, e);
    store_output(p, tg.c, e, v);
    if (tg.add_out != nullptr) tg.add_out[e] = tg.add_src[e] + v;
  }
}

// ---- host side: tile height and ring depth for one launch
struct StagedPlan {
  int rgs;     // row groups per CTA
  int stages;  // ring depth
  size_t smem;
  double cost;  // modelled microseconds
};

inline int device_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    sms = v > 0 ? v : 148;
  }
  return sms;
}

// Four consumer sets pay off when 64-row tiles would leave a good part of the SMs without a
// CTA (measured: 80 and 68 CTAs on 148 SMs gain 0.5-1 us, 136 CTAs gain nothing).
inline bool four_sets_worthwhile(uint64_t n, uint64_t split) {
  return ((n + 63) / 64) * split * 10 <= static_cast<uint64_t>(device_sms()) * 6;
}

// Picks the tile height (16..64 rows) and the CTAs per SM so that the grid is
// one wave with as even a load per SM as the shape allows.  The model: a CTA
// costs a fixed prefix (launch, activation staging, epilogue) plus time
// proportional to its rows x blocks, SMs work through their CTAs at a fixed
// rate, and every further wave pays the prefix again.
//   fixed(rgs)      shared memory besides the ring, in bytes
//   stage_bytes(rgs) one ring stage
template <typename FixedFn, typename StageFn>
inline bool plan_staged(uint64_t n, uint64_t split, uint64_t per, uint64_t nchunks, int max_want,
                        int regs_per_thread, FixedFn fixed, StageFn stage_bytes, StagedPlan* out,
                        int sets = 2) {
  const int sms = device_sms();
  // per 16 rows x 1 block on a busy SM; per block of one warp's own chunks; per wave
  const double kUnitUs = 0.04, kWarpBlockUs = 0.5, kPrefixUs = 3.4;
  double best = 1e30;
  bool found = false;
  for (int rgs = 4; rgs >= 1; --rgs) {
    const uint64_t th = 16u * rgs;
    const uint64_t ctas = ((n + th - 1) / th) * split;
    const size_t fx = fixed(rgs), sb = stage_bytes(rgs);
    for (int occ = 1; occ <= 4; ++occ) {
      if (occ > 1 && occ * (sets * rgs + 1) * 32 * regs_per_thread > 65536) break;  // register file
      const size_t avail = static_cast<size_t>(kMaxSmem) / occ;
      const size_t reserve = occ > 1 ? 1024 : 0;  // per-CTA reservation of the hardware
      if (avail < fx + reserve + sets * sb) break;  // every consumer set owns at least one slot
      int depth = static_cast<int>((avail - reserve - fx) / sb);
      int want = static_cast<int>(nchunks < static_cast<uint64_t>(max_want) ? nchunks : max_want);
      if (want < sets) want = sets;
      if (depth > want) depth = want;
      const uint64_t slots = static_cast<uint64_t>(sms) * occ;
      const uint64_t waves = (ctas + slots - 1) / slots;
      const uint64_t per_sm = (ctas + sms - 1) / sms;
      // an SM works through its CTAs at a fixed rate, but a warp cannot go faster
      // than its own share of the blocks (one consumer set's) one after the other
      const double throughput = per_sm * rgs * per * kUnitUs;
      const double latency = waves * (static_cast<double>(per) / sets) * kWarpBlockUs;
      double cost = (throughput > latency ? throughput : latency) + waves * kPrefixUs;
      if (depth < sets + 1 && nchunks > static_cast<uint64_t>(sets)) cost *= 1.1;  // a shallow ring stalls on HBM latency
      if (cost < best - 1e-9) {
        best = cost;
        out->rgs = rgs;
        out->stages = depth;
        out->smem = fx + static_cast<size_t>(depth) * sb;
        out->cost = cost;
        found = true;
      }
    }
  }
  return found;
}

// ---- launch plan of the multi-target kernels (Q4_K, Q6_K)
struct GroupPlan {
  int rgs, stages, sets, split, grid_x, occ;
  bool cluster;  // split > 1 inside the launch: the chunks of a tile form a cluster (else: tickets)
  size_t smem;
  double cost;  // modelled microseconds
};

inline int env_plan_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}

// Picks the tile height, the CTAs per SM, the ring depth and (when the split is
// the launch's own business, fixed_split == 0) the number of k chunks for a
// launch over `count` weight tensors of n[i] rows and nb blocks per row.  The
// grid is never larger than the SMs can hold at once: a CTA works through
// several tiles instead, so the activation staging is paid once per CTA.
//   fixed(rgs, per)   shared memory besides the ring, in bytes, for `per` blocks per chunk
//   stage_bytes(rgs)  one ring stage
//   nchunks(per)      ring stages one tile of `per` blocks needs
template <typename FixedFn, typename StageFn, typename ChunksFn>
inline bool plan_group(const uint64_t* n, int count, uint64_t nb, int m, uint64_t fixed_split, int sets,
                       int fixed_rgs, int regs_per_thread, int max_want, double block_us, FixedFn fixed,
                       StageFn stage_bytes, ChunksFn nchunks, GroupPlan* out, bool allow_cluster = true) {
  const int sms = device_sms();
  // Measured on B200 (Q4_K, m = 1): a busy SM gets through one 16-row x 256-column block in
  // about 0.053 us whatever the tiling; one warp needs `block_us` (0.5 us Q4_K) for each block
  // of its own chain; every tile of a CTA ends with about 0.5 us of exchange and output; a
  // launch costs about 2.6 us before and after its weights, plus the
  // activation staging (0.25 us per round of one block per consumer warp); a split inside the
  // launch pays a ticket round trip and a pass over the partial sums at the very end of every
  // tile, where nothing overlaps it (measured 3-4 us: no cheaper than a reduce launch, so it
  // only wins where it shortens a long chain, as for Q6_K rows of 68 blocks).
  const double kUnitUs = 0.053 * (block_us / 0.5), kPrefixUs = 2.6, kStageRoundUs = 0.25;
  const double kTicketUs = 3.5, kTicketTileUs = 1.5, kWaveUs = 2.0, kTileUs = 0.5;
  const double kClusterUs = env_plan_int("TSR_CLUSTER_NS", 1000) * 1e-3, kClusterTileUs = 0.3;
  // Off unless TSR_CLUSTER=1: measured on B200 the cluster plans this model prefers (5120 rows,
  // k = 17408 / 6144: 48-row tiles, four chunks, three CTAs per SM) ran 5-9 us slower than the
  // unsplit four-set plan (22.7 against 16.9 us, Q6_K 34.8 against 25.8 us): three CTAs per SM
  // leave each consumer set one or two ring slots, which does not cover the HBM latency, and
  // the SMs are no more evenly loaded than with 48-row tiles alone.
  const bool use_cluster = TSR_CLUSTER_SPLIT != 0 && allow_cluster && env_plan_int("TSR_CLUSTER", 0) != 0;
  const int ring_max = env_plan_int("TSR_RING_MAX", max_want);
  const int force_rgs = env_plan_int("TSR_RGS", 0), force_split = env_plan_int("TSR_SPLIT", 0);
  const int force_grid = env_plan_int("TSR_GRID", 0), force_occ = env_plan_int("TSR_OCC", 0);
  const int force_persist = env_plan_int("TSR_PERSIST", -1);
  double best = 1e30;
  bool found = false;
  for (uint64_t split = 1; split <= 8 && split <= nb; ++split) {
    if (fixed_split != 0 && split != fixed_split) continue;
    if (fixed_split == 0 && force_split > 0 && split != static_cast<uint64_t>(force_split)) continue;
    if (nb % split != 0) continue;
    const uint64_t per = nb / split;
    const uint64_t chunks_per_tile = nchunks(per);
    for (int rgs = 4; rgs >= 1; --rgs) {
      if (fixed_rgs != 0 && rgs != fixed_rgs) continue;
      if (fixed_rgs == 0 && force_rgs >= 1 && force_rgs <= 4 && rgs != force_rgs) continue;
      const uint64_t th = 16u * rgs;
      uint64_t tiles = 0;
      for (int i = 0; i < count; ++i) tiles += (n[i] + th - 1) / th;
      const size_t fx = fixed(rgs, per), sb = stage_bytes(rgs);
      const int warps = sets * rgs;
      for (int occ = 1; occ <= 4; ++occ) {
        if (force_occ > 0 && occ != force_occ) continue;
        if (occ > 1 && occ * (warps + 1) * 32 * regs_per_thread > 65536) break;  // register file
        if (occ > 1 && sets == 4) break;  // the four-set kernels are built for one CTA per SM
        const size_t avail = static_cast<size_t>(kMaxSmem) / occ;
        const size_t reserve = occ > 1 ? 1024 : 0;  // per-CTA reservation of the hardware
        if (avail < fx + reserve + sets * sb) break;  // every consumer set owns at least one slot
        const uint64_t slots = static_cast<uint64_t>(sms) * occ;
        // a grid the SMs hold at once, each CTA working through several tiles -- or, when that
        // would be at most two rounds, one CTA per tile (no tile loop, but a second prefix)
        for (int persist = 1; persist >= 0; --persist) {
          if (force_persist >= 0 && persist != force_persist) continue;
          uint64_t grid_x = slots / split;
          if (grid_x == 0) grid_x = 1;
          if (grid_x > tiles) grid_x = tiles;
          if (!persist) {
            if (grid_x == tiles || tiles * split > 2 * slots) continue;  // same plan, or too many rounds
            grid_x = tiles;
          }
          if (force_grid > 0) grid_x = static_cast<uint64_t>(force_grid) < tiles ? force_grid : tiles;
          const uint64_t tiles_per_cta = (tiles + grid_x - 1) / grid_x;
          const uint64_t total_chunks = tiles_per_cta * chunks_per_tile;
          int depth = static_cast<int>((avail - reserve - fx) / sb);
          int want = static_cast<int>(total_chunks < static_cast<uint64_t>(ring_max) ? total_chunks : ring_max);
          if (want < sets) want = sets;
          if (depth > want) depth = want;
          const uint64_t ctas = grid_x * split;
          const uint64_t waves = (ctas + slots - 1) / slots;
          const uint64_t ctas_per_sm = (ctas + sms - 1) / sms;
          // an SM works through its CTAs' tiles at a fixed rate, but a warp cannot go faster
          // than its own share of the blocks (one consumer set's) one after the other
          // (four sets spend a little more on adding their partial sums per tile)
          const double throughput =
              static_cast<double>(ctas_per_sm * tiles_per_cta * rgs * per) * kUnitUs * (sets == 4 ? 1.05 : 1.0);
          const double chain = static_cast<double>(waves * tiles_per_cta) * ((per + sets - 1) / sets) * block_us;
          const double staging = kStageRoundUs * static_cast<double>((m * per + warps - 1) / warps);
          // every tile of a CTA ends with the exchange between the sets and the output pass
          double cost = kPrefixUs + staging + (throughput > chain ? throughput : chain) + (waves - 1) * kWaveUs +
                        kTileUs * static_cast<double>(waves * tiles_per_cta) + (sets == 4 ? 0.4 : 0.0);
          // the chunks of a tile meet through the shared memory of a cluster where a CTA has few
          // enough tiles for its receive buffers, else through tickets in global memory
          const bool cluster = split > 1 && fixed_split == 0 && tiles_per_cta <= static_cast<uint64_t>(kClusterTiles) &&
                               use_cluster;
          if (split > 1 && fixed_split == 0)
            cost += cluster ? kClusterUs + kClusterTileUs * static_cast<double>(tiles_per_cta)
                            : kTicketUs + kTicketTileUs * static_cast<double>(tiles_per_cta);
          if (depth < sets + 1 && total_chunks > static_cast<uint64_t>(sets)) cost *= 1.1;  // a shallow ring stalls on HBM latency
          if (cost < best - 1e-9) {
            best = cost;
            out->rgs = rgs;
            out->stages = depth;
            out->sets = sets;
            out->split = static_cast<int>(split);
            out->grid_x = static_cast<int>(grid_x);
            out->occ = occ;
            out->cluster = cluster;
            out->smem = fx + static_cast<size_t>(depth) * sb;
            out->cost = cost;
            found = true;
          }
        }
      }
    }
  }
  if (found && env_plan_int("TSR_PLAN_DEBUG", 0))
    std::fprintf(stderr, "plan: targets %d nb %llu sets %d -> rgs %d occ %d split %d%s grid_x %d stages %d smem %zu cost %.1f us\n",
                 count, static_cast<unsigned long long>(nb), sets, out->rgs, out->occ, out->split,
                 out->cluster ? " (cluster)" : "", out->grid_x, out->stages, out->smem, out->cost);
  return found;
}

// plan_group with a memo: a launch's plan depends only on its shape, the kernel variant (`tag`,
// unique per kernel instantiation) and the experiment switches, and the same few shapes come
// back for every token.  Not used while TSR_PLAN_DEBUG is set (the plan prints as it is made).
template <typename FixedFn, typename StageFn, typename ChunksFn>
inline bool plan_group_cached(int tag, const uint64_t* n, int count, uint64_t nb, int m, uint64_t fixed_split, int sets,
                              int fixed_rgs, int regs_per_thread, int max_want, double block_us, FixedFn fixed,
                              StageFn stage_bytes, ChunksFn nchunks, GroupPlan* out, bool allow_cluster = true) {
  if (env_plan_int("TSR_PLAN_DEBUG", 0))
    return plan_group(n, count, nb, m, fixed_split, sets, fixed_rgs, regs_per_thread, max_want, block_us, fixed,
                      stage_bytes, nchunks, out, allow_cluster);
  struct Entry {
    uint64_t key[12];
    bool ok;
    GroupPlan plan;
  };
  uint64_t key[12] = {};
  for (int i = 0; i < count && i < 4; ++i) key[i] = n[i];
  key[4] = (static_cast<uint64_t>(tag) << 40) | (static_cast<uint64_t>(count) << 32) | (static_cast<uint64_t>(sets) << 24) |
           (static_cast<uint64_t>(fixed_rgs) << 16) | (allow_cluster ? 1u : 0u);
  key[5] = nb;
  key[6] = (static_cast<uint64_t>(m) << 32) | fixed_split;
  key[7] = (static_cast<uint64_t>(static_cast<uint32_t>(env_plan_int("TSR_RING_MAX", max_want))) << 32) |
           static_cast<uint32_t>(env_plan_int("TSR_RGS", 0));
  key[8] = (static_cast<uint64_t>(static_cast<uint32_t>(env_plan_int("TSR_SPLIT", 0))) << 32) |
           static_cast<uint32_t>(env_plan_int("TSR_GRID", 0));
  key[9] = (static_cast<uint64_t>(static_cast<uint32_t>(env_plan_int("TSR_OCC", 0))) << 32) |
           static_cast<uint32_t>(env_plan_int("TSR_PERSIST", -1));
  key[10] = (static_cast<uint64_t>(static_cast<uint32_t>(env_plan_int("TSR_CLUSTER", 0))) << 32) |
            static_cast<uint32_t>(env_plan_int("TSR_CLUSTER_NS", 1000));
  int dev = 0;
  cudaGetDevice(&dev);
  key[11] = (static_cast<uint64_t>(static_cast<uint32_t>(dev)) << 32) | static_cast<uint32_t>(regs_per_thread);
  static std::mutex mutex;
  static std::vector<Entry> cache;
  {
    std::lock_guard<std::mutex> lock(mutex);
    for (const Entry& e : cache) {
      bool same = true;
      for (int i = 0; i < 12; ++i) same = same && e.key[i] == key[i];
      if (same) {
        *out = e.plan;
        return e.ok;
      }
    }
  }
  Entry e{};
  for (int i = 0; i < 12; ++i) e.key[i] = key[i];
  e.ok = plan_group(n, count, nb, m, fixed_split, sets, fixed_rgs, regs_per_thread, max_want, block_us, fixed, stage_bytes,
                    nchunks, &e.plan, allow_cluster);
  *out = e.plan;
  std::lock_guard<std::mutex> lock(mutex);
  if (cache.size() < 4096) cache.push_back(e);
  return e.ok;
}

// How many clusters of `cluster_y` CTAs of `kernel` the device holds at once with this block
// size and shared memory (0: such a cluster cannot be launched).  Cached per configuration.
template <typename Kernel>
inline int max_active_clusters(Kernel kernel, int threads, size_t smem, int cluster_y) {
  struct Key {
    const void* k;
    int dev, threads, cluster;
    size_t smem;
    int result;
  };
  static std::mutex mutex;
  static std::vector<Key> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mutex);
  for (const Key& e : cache)
    if (e.k == reinterpret_cast<const void*>(kernel) && e.dev == dev && e.threads == threads && e.cluster == cluster_y &&
        e.smem == smem)
      return e.result;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, static_cast<unsigned>(cluster_y));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(cluster_y);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(kernel), &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  cache.push_back(Key{reinterpret_cast<const void*>(kernel), dev, threads, cluster_y, smem, n});
  return n;
}

// Registers per thread of a kernel, rounded up to the allocation unit.
template <typename Kernel>
inline int kernel_registers(Kernel kernel) {
  cudaFuncAttributes attr{};
  if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess || attr.numRegs <= 0) return 128;
  return (attr.numRegs + 7) & ~7;
}

}  // namespace staged
}  // namespace tsr
