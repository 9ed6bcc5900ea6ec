// tcgen05 tiles that read the weights straight from shared memory, for batches of
// 2..21 activation rows:
//   FP8 E4M3 weights, kind::f8f6f4: C[m,n] = A[m,k] . (s[n] * e4m3(W[n,k]))^T, the contract of
//     the reference's gemm_fp8 (src/backends/vulkan/kernels/gemm_fp8.comp:52-68; GemmFp8Ref,
//     src/core/numerics/gemm.cpp:253-277 of the reference);
//   MXFP4 weights (E2M1 nibbles, one E8M0 scale per 32), kind::mxf8f6f4.block_scale: the
//     contract of gemm_mxfp4 / _rows / _batched (gemm_mxfp4.comp:51-87; GemmMxFp4Ref,
//     gemm.cpp:311-344) and, with E4M3 activation codes and per-row scales handed in, of
//     gemm_mxfp4_wmma (gemm_mxfp4_wmma.comp:78-117).  The TMA unpacks the nibbles on the fly
//     (16 nibbles per 16-byte piece of shared memory, the layout kind::mxf8f6f4 reads 4-bit
//     operands in); the weights' own E8M0 bytes are the A-side scale factors of the MMA: the
//     epilogue warps fetch the CTA's part of the side table once, re-lay each 128-row x 128-k
//     group as 32 rows of 16 bytes (row r: the four scales of rows r, r + 32, r + 64, r + 96)
//     and the MMA warp copies it into tensor memory with tcgen05.cp.32x128b.warpx4; the B-side
//     scale factors are all 1.
//
// The weight bytes are the tensor core's A operand exactly as they lie in HBM:
// a TMA box of 128 rows x 128 bytes lands in shared memory in the 128-byte
// swizzled K-major layout that tcgen05.mma reads, so no thread ever touches a
// weight.  The activations are the B operand: each fp32 row is split once per
// launch into three E4M3 terms x ~ s1*(t1 + t2/16 + t3/256) (s1 = row maximum /
// 448; every term is the E4M3 rounding of what the earlier terms left over, so
// an element keeps 12 significant bits), one column of B per (row, term); the
// epilogue adds the three accumulator columns of a row with their weights and
// applies the weight row scale.  E4M3 x E4M3 products are exact in the fp32
// accumulator, so the only rounding is that of the activations.
//
// Per CTA: 128 weight rows, one range of k; warp 0 issues the TMA copies of a
// four-stage ring (two 128-byte k segments of weights and of activation terms
// per stage), warp 1 issues eight K = 32 MMAs per stage into TMEM and commits
// them to the stage's empty barrier, warps 2-5 read the accumulator with
// tcgen05.ld and store C (or this CTA's partial sums when k is split over
// CTAs; the regions are then added in order by the reduce kernel).  Every
// wait is bounded and TMEM is released on every path.
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "codec.cuh"
#include "launch.h"
#include "pipeline.cuh"
#include "tessera_b200.h"

namespace tsr {

__device__ unsigned int g_f8_timeouts = 0;

namespace {

constexpr int kTileM = 128;     // weight rows per CTA
constexpr int kSegBytes = 128;  // k elements (bytes) per shared-memory row: one swizzle span
constexpr int kSegs = 2;        // segments per stage
constexpr int kMaxStages = 4;
constexpr int kTerms = 3;
constexpr int kMaxCols = 64;  // B columns (activation rows x terms, padded to 16)
constexpr int kThreads = 6 * 32;
constexpr int kWeightStage = kSegs * kTileM * kSegBytes;  // 32 KiB

enum : int { kFp8 = 0, kMxFp4 = 1 };

struct F8Params {
  const float* row_scale;  // [n] (FP8) or null
  const float* term_scale;  // [m]: s1 of each activation row
  float* out;               // C, or partial regions [split][m][n]
  int m, n, k;
  int ncols;       // B columns, a multiple of 16
  int stages_per_cta;
  int total_stages;
  int ring;  // stages of the shared-memory ring (2..4)
  int pdl;   // launched as a programmatic dependent of the kernel that writes the activation terms
  int terms;  // B columns per activation row: 3 (fp32 activations split here) or 1 (E4M3 codes handed in)
  const unsigned char* sf;  // MXFP4: the E8M0 side table, n rows of k / 32 bytes
};

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{.reg .pred p; setp.ne.b32 p, %4, 0; "
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Block-scaled form: sfa / sfb are tensor-memory column addresses of the scale factors (one
// 32-bit column per 32 rows holds four consecutive K blocks; the descriptor's sf ids pick the byte).
__device__ __forceinline__ void umma_mxf8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{.reg .pred p; setp.ne.b32 p, %6, 0; "
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
// 32 rows x 16 bytes of shared memory into the same four columns of all four lane quadrants.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with
// the 128-byte swizzle (what a TMA box with CU_TENSOR_MAP_SWIZZLE_128B writes): eight rows
// form a 1024-byte group (stride byte offset), the leading byte offset is not used by
// swizzled K-major layouts, descriptor version 1, layout type 2.  The tile must start on a
// 1024-byte boundary; a K step inside the row advances the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Descriptor of a scale-factor piece: 32 rows of 16 bytes, no swizzle, K-major; the 8-row
// groups are 128 bytes apart (stride byte offset), one 16-byte column only.
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((128 >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  return d;
}
// kind::mxf8f6f4.block_scale: D fp32, A E2M1 (format 5), B E4M3 (0), both K-major, E8M0
// scale factors, M = 128, N = n_cols; a_sf = byte of the scale-factor column this K block uses.
__device__ __forceinline__ uint32_t instr_desc_mx(uint32_t n_cols, uint32_t a_sf) {
  return (5u << 7) | ((n_cols >> 3) << 17) | (1u << 23) | ((kTileM >> 4) << 24) | (a_sf << 29);
}

// kind::f8f6f4: D fp32, A and B E4M3 (format 0), both K-major, M = 128, N = n_cols.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n_cols) {
  return (1u << 4) | ((n_cols >> 3) << 17) | ((kTileM >> 4) << 24);
}

__device__ __forceinline__ float e4m3_round(float v, uint32_t* code) {
  const __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  *code = c;
  return e4m3_to_float(c);
}

// Column 3 t + j of B holds term j of activation row t (zeros beyond m); b: [ncols][k]
// bytes; term_scale[t] = s1 of row t.  CTA (x, y): k elements [1024 y, 1024 y + 1024) of
// activation row x, all three terms; rows beyond m are the zero columns that pad B to a
// multiple of 16.  Every CTA of a row finds the row maximum by itself (the row is a few
// tens of KB, served from L2).
constexpr int kTermChunk = 1024;
__global__ void __launch_bounds__(256)
activation_terms_kernel(const float* __restrict__ a, unsigned char* __restrict__ b, float* __restrict__ term_scale,
                        int m, int k, int ncols) {
  __shared__ float red[8];
  pdl_wait();     // the activations may come from the kernel just ahead
  pdl_trigger();  // the tile kernel may start fetching weights
  const int t = blockIdx.x, k0 = blockIdx.y * kTermChunk;
  if (t >= m) {
    // zero columns 3 m .. ncols - 1: CTA (m + i, y) clears column 3 m + i
    const int col = kTerms * m + (t - m);
    if (col < ncols)
      for (int i = k0 + threadIdx.x * 16; i < min(k, k0 + kTermChunk); i += 256 * 16)
        *reinterpret_cast<uint4*>(b + static_cast<size_t>(col) * k + i) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const float* src = a + static_cast<size_t>(t) * k;
  float amax = 0.0f;
  for (int i = threadIdx.x * 4; i < k; i += 256 * 4) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(src + i));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  // a power of two, so the scalings below are exact; 256 <= 448: the largest element is in range
  const float s1 = fminf(fmaxf(exp2f(ceilf(log2f(fmaxf(amax, 1e-30f))) - 8.0f), 1e-30f), 1e30f);
  if (blockIdx.y == 0 && threadIdx.x == 0) term_scale[t] = s1;
  const float inv1 = 1.0f / s1;
  const int i0 = k0 + threadIdx.x * 4;
  if (i0 < k) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(src + i0));
    const float xs[4] = {x.x, x.y, x.z, x.w};
    uint32_t w1 = 0, w2 = 0, w3 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t c1, c2, c3;
      const float v = xs[j] * inv1;               // |v| <= 256
      const float r1 = v - e4m3_round(v, &c1);    // exact: v and its rounding are close
      const float r2 = r1 * 16.0f;
      const float r3 = (r2 - e4m3_round(r2, &c2)) * 16.0f;
      e4m3_round(r3, &c3);
      w1 |= c1 << (8 * j);
      w2 |= c2 << (8 * j);
      w3 |= c3 << (8 * j);
    }
    unsigned char* dst = b + static_cast<size_t>(kTerms * t) * k + i0;
    *reinterpret_cast<uint32_t*>(dst) = w1;
    *reinterpret_cast<uint32_t*>(dst + k) = w2;
    *reinterpret_cast<uint32_t*>(dst + 2 * static_cast<size_t>(k)) = w3;
  }
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, 2)
gemm_f8_umma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap bmap,
                    const F8Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b_stage = kSegs * p.ncols * kSegBytes;
  const int kStages = p.ring;
  unsigned char* const w_tiles = smem;                          // [ring][kSegs][128 rows][128 B]
  unsigned char* const b_tiles = smem + kStages * kWeightStage;  // [ring][kSegs][ncols][128 B]
  uint64_t* full = reinterpret_cast<uint64_t*>(b_tiles + kStages * b_stage);
  uint64_t* empty = full + kMaxStages;
  uint64_t* done = empty + kMaxStages;
  uint64_t* sf_full = done + 1;  // [kMaxStages] scale factors of a stage are in shared memory (MXFP4)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_full + kMaxStages);
  // MXFP4 only: [ring][kSegs][512 B] scale factors in tcgen05.cp order, then 512 B of 1.0 for the B side
  unsigned char* const sf_stage = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tmem_slot + 4) + 127) & ~uintptr_t(127));  // descriptors address 16-byte units
  unsigned char* const sf_ones = sf_stage + kMaxStages * kSegs * 512;
  const int row0 = blockIdx.x * kTileM;
  const int stage0 = blockIdx.y * p.stages_per_cta;
  const int nstages = min(p.stages_per_cta, p.total_stages - stage0);
  // tensor memory: the accumulator, then (MXFP4) four scale-factor columns per segment of
  // every ring stage and four for the B side
  const uint32_t sfa_col = static_cast<uint32_t>(p.ncols), sfb_col = sfa_col + kMaxStages * kSegs * 4;
  uint32_t tmem_cols = 32;
  while (tmem_cols < (FMT == kMxFp4 ? sfb_col + 4 : static_cast<uint32_t>(p.ncols))) tmem_cols <<= 1;

  if (tid == 0) {
    tma_prefetch_descriptor(&wmap);
    tma_prefetch_descriptor(&bmap);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&sf_full[s], 4);  // one arrival per epilogue warp
    }
    mbar_init(done, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (p.pdl && warp != 0) {
    // everything these warps read or write after this point may depend on the kernel ahead
    pdl_wait();
  }
  if (tid == 32) pdl_trigger();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA issuer ------------------------------------------------
      // a copy of packed nibbles counts the bytes it reads, not the padded bytes it writes
      const uint32_t bytes = static_cast<uint32_t>((FMT == kMxFp4 ? kWeightStage / 2 : kWeightStage) + b_stage);
      // The weights do not depend on the kernel ahead (which writes the activation terms):
      // the first ring of weight stages is on its way before the wait for that kernel.
      const int first = nstages < kStages ? nstages : kStages;
      for (int s = 0; s < first; ++s) {
        mbar_expect_tx(&full[s], bytes);
        // (128 B, rows, segments): two consecutive k segments per stage
        tma_load_3d(w_tiles + s * kWeightStage, &wmap, 0, row0, kSegs * (stage0 + s), &full[s]);
      }
      if (p.pdl) pdl_wait();
      for (int s = 0; s < first; ++s) tma_load_3d(b_tiles + s * b_stage, &bmap, 0, 0, kSegs * (stage0 + s), &full[s]);
      for (int s = first; s < nstages; ++s) {
        const int slot = s % kStages, round = s / kStages;
        if (!mbar_wait(&empty[slot], (round - 1) & 1, &g_f8_timeouts)) break;
        mbar_expect_tx(&full[slot], bytes);
        tma_load_3d(w_tiles + slot * kWeightStage, &wmap, 0, row0, kSegs * (stage0 + s), &full[slot]);
        tma_load_3d(b_tiles + slot * b_stage, &bmap, 0, 0, kSegs * (stage0 + s), &full[slot]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ------------------------------------------------
      const uint32_t idesc = instr_desc(static_cast<uint32_t>(p.ncols));
      bool ok = true;
      for (int s = 0; s < nstages; ++s) {
        const int slot = s % kStages, round = s / kStages;
        if (!mbar_wait(&full[slot], round & 1, &g_f8_timeouts) ||
            (FMT == kMxFp4 && !mbar_wait(&sf_full[slot], round & 1, &g_f8_timeouts))) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(w_tiles + slot * kWeightStage), b_addr = smem_u32(b_tiles + slot * b_stage);
        if (FMT == kMxFp4) {
          if (s == 0) tmem_cp_32x128b_x4(tmem_base + sfb_col, smem_desc_sf(smem_u32(sf_ones)));
#pragma unroll
          for (int seg = 0; seg < kSegs; ++seg)
            tmem_cp_32x128b_x4(tmem_base + sfa_col + (slot * kSegs + seg) * 4,
                               smem_desc_sf(smem_u32(sf_stage + (slot * kSegs + seg) * 512)));
        }
#pragma unroll
        for (int seg = 0; seg < kSegs; ++seg) {
#pragma unroll
          for (int kk = 0; kk < kSegBytes / 32; ++kk) {
            const uint64_t adesc = smem_desc_sw128(a_addr + seg * kTileM * kSegBytes + kk * 32);
            const uint64_t bdesc = smem_desc_sw128(b_addr + seg * p.ncols * kSegBytes + kk * 32);
            const uint32_t acc = (s > 0 || seg > 0 || kk > 0) ? 1u : 0u;
            if (FMT == kMxFp4) {
              umma_mxf8f6f4(tmem_base, adesc, bdesc, instr_desc_mx(static_cast<uint32_t>(p.ncols), kk),
                            tmem_base + sfa_col + (slot * kSegs + seg) * 4, tmem_base + sfb_col, acc);
            } else {
              umma_f8(tmem_base, adesc, bdesc, idesc, acc);
            }
          }
        }
        umma_commit(&empty[slot]);  // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(done);
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> C -----------------------------
    // a warp reads the TMEM lanes of its quadrant (warp index mod 4)
    const int quad = warp & 3;
    if (FMT == kMxFp4) {
      // First the scale factors: thread t serves weight row row0 + t.  Stage by stage it writes the
      // row's scale word of each segment (four E8M0 bytes, one per K block of 32) where
      // tcgen05.cp.32x128b.warpx4 wants it: row t % 32 of the 512-byte piece, word t / 32.  The
      // words come straight from the side table, a few stages ahead of their use.
      const int et = tid - 64;  // 0..127
      const int grow = row0 + et;
      const int sf_words = p.k / 128;  // scale words per weight row
      const uint32_t* sf_row = reinterpret_cast<const uint32_t*>(p.sf + static_cast<size_t>(grow < p.n ? grow : 0) * (p.k / 32));
      auto fetch = [&](int s, int seg) -> uint32_t {
        const int wd = (stage0 + s) * kSegs + seg;
        // rows beyond n and segments beyond k multiply zero weights: any finite scale will do
        return (s < nstages && grow < p.n && wd < sf_words) ? __ldg(sf_row + wd) : 0x7F7F7F7Fu;
      };
      constexpr int kAhead = 4;
      uint32_t pre[kAhead][kSegs];
#pragma unroll
      for (int u = 0; u < kAhead; ++u)
#pragma unroll
        for (int seg = 0; seg < kSegs; ++seg) pre[u][seg] = fetch(u, seg);
      if (et < 128) reinterpret_cast<uint32_t*>(sf_ones)[et] = 0x7F7F7F7Fu;
      for (int s0 = 0; s0 < nstages; s0 += kAhead) {
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
          const int s = s0 + u;
          if (s < nstages) {
            const int slot = s % kStages, round = s / kStages;
            if (round > 0 && !mbar_wait(&empty[slot], (round - 1) & 1, &g_f8_timeouts)) break;
#pragma unroll
            for (int seg = 0; seg < kSegs; ++seg)
              *reinterpret_cast<uint32_t*>(sf_stage + (slot * kSegs + seg) * 512 + (et & 31) * 16 + (et >> 5) * 4) = pre[u][seg];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sf_full[slot]);
#pragma unroll
            for (int seg = 0; seg < kSegs; ++seg) pre[u][seg] = fetch(s + kAhead, seg);
          }
        }
      }
    }
    const bool ok = __all_sync(0xFFFFFFFFu, nstages > 0 && mbar_wait(done, 0, &g_f8_timeouts));
    tcgen05_fence_after();
    if (ok) {
      const int out_row = row0 + quad * 32 + lane;
      const float rs = (FMT == kFp8 && out_row < p.n) ? __ldg(p.row_scale + out_row) : 1.0f;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      float* out = p.out + static_cast<size_t>(blockIdx.y) * p.m * p.n;
      if (p.terms == 1) {
        // one column per activation row (E4M3 codes handed in): scale by the row's own factor
        for (int c0 = 0; c0 < p.ncols; c0 += 8) {
          float d[8];
          tmem_ld8(lane_addr + c0, d);
          if (out_row < p.n) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c0 + j < p.m) out[static_cast<size_t>(c0 + j) * p.n + out_row] = d[j] * __ldg(p.term_scale + c0 + j) * rs;
          }
        }
      } else
      // 24 columns = 8 activation rows at a time
      for (int c0 = 0; c0 < p.ncols; c0 += 24) {
        float d[24];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          if (c0 + 8 * q < p.ncols) {
            tmem_ld8(lane_addr + c0 + 8 * q, d + 8 * q);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) d[8 * q + j] = 0.0f;
          }
        }
        if (out_row < p.n) {
#pragma unroll
          for (int tt = 0; tt < 8; ++tt) {
            const int t = c0 / kTerms + tt;
            if (t < p.m) {
              const float s1 = __ldg(p.term_scale + t);
              const float v = d[3 * tt] + d[3 * tt + 1] * 0.0625f + d[3 * tt + 2] * 0.00390625f;
              out[static_cast<size_t>(t) * p.n + out_row] = v * s1 * rs;
            }
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// ---- tensor maps ------------------------------------------------------------------
struct MapKey {
  const void* base;
  uint64_t rows, k;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && k == o.k && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& x) const {
    return std::hash<const void*>()(x.base) ^ (x.rows * 0x9E3779B97F4A7C15ull) ^ (x.k << 36) ^ (static_cast<size_t>(x.box_rows) << 56);
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// rows x k elements, row-major, as (128 elements, rows, k / 128) with a box of (128, box_rows, 2)
// and the 128-byte swizzle.  nibbles = false: one byte per element.  nibbles = true: packed
// 4-bit elements that the TMA unpacks to 16 per 16-byte piece (the base must be 32-byte aligned).
int matrix_map(const void* base, uint64_t rows, uint64_t k, uint32_t box_rows, bool nibbles, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{base, rows, k | (nibbles ? 1ull << 62 : 0), box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return kOk;
  }
  const uint64_t dims[3] = {kSegBytes, rows, k / kSegBytes};
  const uint64_t strides[2] = {nibbles ? k / 2 : k, static_cast<uint64_t>(nibbles ? kSegBytes / 2 : kSegBytes)};
  const uint32_t box[3] = {kSegBytes, box_rows, kSegs};
  CUtensorMap map;
  const int rc = encode_tensor_map(&map, nibbles ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                                   3, base, dims, strides, box, true);
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


// What the three entry points below share.  fmt kFp8: w = n x k bytes, scale = row scales.
// fmt kMxFp4: w = nibbles then E8M0 side table.  codes == null: a = fp32 activations, split here
// into three E4M3 terms; codes != null: E4M3 activation codes (m x k bytes) with their per-row
// factors `code_scale`, used as they are (one B column per row).
int launch_tile(int fmt, const float* a, const unsigned char* codes, const float* code_scale, const void* w,
                const float* scale, float* c, uint64_t m, uint64_t n, uint64_t k, cudaStream_t st) {
  const int terms = codes != nullptr ? 1 : kTerms;
  const uint64_t ncols = (m * terms + 15) / 16 * 16;
  if (ncols > kMaxCols || k % kSegBytes != 0 || k < 2 * kSegBytes || (reinterpret_cast<uintptr_t>(w) & 31u) ||
      (codes != nullptr && (reinterpret_cast<uintptr_t>(codes) & 15u)) || env_int("TSR_DISABLE_F8_UMMA", 0))
    return kUnsupportedFeature;
  const uint64_t total_stages = (k / kSegBytes + kSegs - 1) / kSegs;
  const uint64_t tiles = (n + kTileM - 1) / kTileM;
  static const int sms = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  // Two CTAs per SM where the ring can be kept at two stages or more; k is split over CTAs
  // until the device is about full (a CTA wants at least three stages of its own).
  const size_t stage_bytes = kWeightStage + kSegs * ncols * kSegBytes;
  const size_t fixed = 1024 + 256 + (fmt == kMxFp4 ? 128 + kMaxStages * kSegs * 512 + 512 : 0);
  int ring = static_cast<int>((227 * 1024 / 2 - 1024 - fixed) / stage_bytes);
  if (ring > kMaxStages) ring = kMaxStages;
  if (ring < 2) return kUnsupportedFeature;
  const uint64_t slots = 2ull * sms;
  uint64_t split = 1;
  const int forced = env_int("TSR_F8_SPLIT", 0);
  while (forced == 0 && tiles * (split + 1) <= slots && total_stages / (split + 1) >= 3) ++split;
  if (forced > 0) split = static_cast<uint64_t>(forced);
  const uint64_t stages_per_cta = (total_stages + split - 1) / split;
  split = (total_stages + stages_per_cta - 1) / stages_per_cta;
  // scratch: B columns (when they are made here), term scales, partial regions.  B rows handed in
  // by the caller are read in place; rows m .. ncols - 1 of the box then lie beyond the tensor
  // and the TMA fills them with zeros.
  const size_t b_bytes = codes != nullptr ? 0 : ncols * k, ts_off = (b_bytes + 255) / 256 * 256, part_off = ts_off + 256;
  const size_t need = part_off + (split > 1 ? split * m * n * 4 : 0);
  unsigned char* scratch = stream_scratch(st, need);
  if (scratch == nullptr) return kUnsupportedFeature;
  float* term_scale = reinterpret_cast<float*>(scratch + ts_off);
  float* part = reinterpret_cast<float*>(scratch + part_off);
  CUtensorMap wmap, bmap;
  if (int rc = matrix_map(w, n, k, kTileM, fmt == kMxFp4, &wmap)) return rc;
  if (codes != nullptr) {
    if (int rc = matrix_map(codes, m, k, static_cast<uint32_t>(ncols), false, &bmap)) return rc;
  } else {
    if (int rc = matrix_map(scratch, ncols, k, static_cast<uint32_t>(ncols), false, &bmap)) return rc;
    const unsigned pad_cols = static_cast<unsigned>(ncols - m * kTerms);
    const bool pdl_terms = pdl_allowed(st, nullptr, 0, scratch, need);
    launch_kernel(activation_terms_kernel,
                  dim3(static_cast<unsigned>(m) + pad_cols, static_cast<unsigned>((k + kTermChunk - 1) / kTermChunk)),
                  dim3(256), 0, st, pdl_terms, a, scratch, term_scale, static_cast<int>(m), static_cast<int>(k),
                  static_cast<int>(ncols));
    if (int rc = check_launch()) return rc;
  }
  const unsigned char* sf = fmt == kMxFp4 ? static_cast<const unsigned char*>(w) + n * (k / 2) : nullptr;
  F8Params p{scale, codes != nullptr ? code_scale : term_scale, split > 1 ? part : c, static_cast<int>(m),
             static_cast<int>(n), static_cast<int>(k), static_cast<int>(ncols), static_cast<int>(stages_per_cta),
             static_cast<int>(total_stages), ring, 1, terms, sf};
  const size_t smem = fixed + static_cast<size_t>(ring) * stage_bytes;
  auto kernel = fmt == kMxFp4 ? gemm_f8_umma_kernel<kMxFp4> : gemm_f8_umma_kernel<kFp8>;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(kernel), 227 * 1024)) return rc;
  // before its wait the tile kernel reads weights only; what runs ahead of it (the terms kernel, or
  // whatever made the codes) does not write them
  const void* wp = w;
  const size_t w_bytes = fmt == kMxFp4 ? n * (k / 2) + n * (k / 32) : n * k;
  const void* outp = split > 1 ? static_cast<const void*>(part) : static_cast<const void*>(c);
  const size_t out_bytes = (split > 1 ? split : 1) * m * n * 4;
  const bool pdl = codes == nullptr ? (pdl_allowed_ranges(st, &wp, &w_bytes, 0, &outp, &out_bytes, 1), true)
                                    : pdl_allowed_ranges(st, &wp, &w_bytes, 1, &outp, &out_bytes, 1);
  p.pdl = pdl ? 1 : 0;
  launch_kernel(kernel, dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(split)), dim3(kThreads), smem, st, pdl,
                wmap, bmap, p);
  if (int rc = check_launch()) return rc;
  if (split > 1) return tsr_gemm_vec_reduce(part, c, m * n, split, st);
  return kOk;
}

}  // namespace

// FP8 weights, 2 <= m <= 21.  kUnsupportedFeature when the shape is outside the tile's range
// or no scratch is to be had (a stream that is being captured before its first plain launch).
int umma_f8_gemm(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n, uint64_t k,
                 cudaStream_t st) {
  if (m < static_cast<uint64_t>(env_int("TSR_TILE_MIN_M", 2)) || k % 16 != 0) return kUnsupportedFeature;
  return launch_tile(kFp8, a, nullptr, nullptr, w, scale, c, m, n, k, st);
}

// MXFP4 weights (nibbles, then the E8M0 side table), fp32 activations, 2 <= m <= 21.
int umma_mxfp4_gemm(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k, cudaStream_t st) {
  if (m < static_cast<uint64_t>(env_int("TSR_TILE_MIN_M", 2)) || env_int("TSR_DISABLE_MX_UMMA", 0)) return kUnsupportedFeature;
  return launch_tile(kMxFp4, a, nullptr, nullptr, w, nullptr, c, m, n, k, st);
}

// MXFP4 weights with E4M3 activation codes (m x k bytes) and their per-row factors: the W4A8
// projection, C[i, j] = as[i] * sum_t e4m3(a8[i, t]) * mxfp4(W[j, t]), m <= 64.
int umma_mxfp4_w4a8(const void* a8, const float* as, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    cudaStream_t st) {
  if (env_int("TSR_DISABLE_MX_UMMA", 0)) return kUnsupportedFeature;
  return launch_tile(kMxFp4, nullptr, static_cast<const unsigned char*>(a8), as, w, nullptr, c, m, n, k, st);
}

int umma_f8_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_f8_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}
int umma_f8_set_error_word(unsigned int* word) { return set_host_error_word(word); }

}  // namespace tsr
