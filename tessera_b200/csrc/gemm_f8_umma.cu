// tcgen05 tile that reads 8-bit weights straight from shared memory
// (kind::f8f6f4): FP8 E4M3 projections with m = 2..21 activation rows.
//
// C[m,n] = A[m,k] . (s[n] * e4m3(W[n,k]))^T, contract of the reference's gemm_fp8
// (src/backends/vulkan/kernels/gemm_fp8.comp:52-68; GemmFp8Ref,
// src/core/numerics/gemm.cpp:253-277 of the reference).
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

struct F8Params {
  const float* row_scale;  // [n]
  const float* term_scale;  // [m]: s1 of each activation row
  float* out;               // C, or partial regions [split][m][n]
  int m, n, k;
  int ncols;       // B columns, a multiple of 16
  int stages_per_cta;
  int total_stages;
  int ring;  // stages of the shared-memory ring (2..4)
  int pdl;   // launched as a programmatic dependent of the kernel that writes the activation terms
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  const int row0 = blockIdx.x * kTileM;
  const int stage0 = blockIdx.y * p.stages_per_cta;
  const int nstages = min(p.stages_per_cta, p.total_stages - stage0);
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.ncols)) tmem_cols <<= 1;

  if (tid == 0) {
    tma_prefetch_descriptor(&wmap);
    tma_prefetch_descriptor(&bmap);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
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
      const uint32_t bytes = static_cast<uint32_t>(kWeightStage + b_stage);
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
        if (!mbar_wait(&full[slot], round & 1, &g_f8_timeouts)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(w_tiles + slot * kWeightStage), b_addr = smem_u32(b_tiles + slot * b_stage);
#pragma unroll
        for (int seg = 0; seg < kSegs; ++seg) {
#pragma unroll
          for (int kk = 0; kk < kSegBytes / 32; ++kk) {
            umma_f8(tmem_base, smem_desc_sw128(a_addr + seg * kTileM * kSegBytes + kk * 32),
                    smem_desc_sw128(b_addr + seg * p.ncols * kSegBytes + kk * 32), idesc,
                    (s > 0 || seg > 0 || kk > 0) ? 1u : 0u);
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
    const bool ok = __all_sync(0xFFFFFFFFu, nstages > 0 && mbar_wait(done, 0, &g_f8_timeouts));
    tcgen05_fence_after();
    if (ok) {
      const int out_row = row0 + quad * 32 + lane;
      const float rs = out_row < p.n ? __ldg(p.row_scale + out_row) : 0.0f;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      float* out = p.out + static_cast<size_t>(blockIdx.y) * p.m * p.n;
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

// rows x k bytes, row-major: (128 B, rows, k / 128) with a box of (128 B, box_rows, 2), 128-byte swizzle
int byte_matrix_map(const void* base, uint64_t rows, uint64_t k, uint32_t box_rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{base, rows, k, box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return kOk;
  }
  const uint64_t dims[3] = {kSegBytes, rows, k / kSegBytes};
  const uint64_t strides[2] = {k, kSegBytes};
  const uint32_t box[3] = {kSegBytes, box_rows, kSegs};
  CUtensorMap map;
  const int rc = encode_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, true);
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

}  // namespace

// FP8 weights, 2 <= m <= 21.  kUnsupportedFeature when the shape is outside the tile's range
// or no scratch is to be had (a stream that is being captured before its first plain launch).
int umma_f8_gemm(const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n, uint64_t k,
                 cudaStream_t st) {
  const uint64_t ncols = (m * kTerms + 15) / 16 * 16;
  if (m < 2 || ncols > kMaxCols || k % kSegBytes != 0 || k < 2 * kSegBytes || k % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(w) & 15u) || env_int("TSR_DISABLE_F8_UMMA", 0))
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
  int ring = static_cast<int>((227 * 1024 / 2 - 3072) / stage_bytes);
  if (ring > kMaxStages) ring = kMaxStages;
  if (ring < 2) return kUnsupportedFeature;
  const uint64_t slots = 2ull * sms;
  uint64_t split = 1;
  const int forced = env_int("TSR_F8_SPLIT", 0);
  while (forced == 0 && tiles * (split + 1) <= slots && total_stages / (split + 1) >= 3) ++split;
  if (forced > 0) split = static_cast<uint64_t>(forced);
  const uint64_t stages_per_cta = (total_stages + split - 1) / split;
  split = (total_stages + stages_per_cta - 1) / stages_per_cta;
  // scratch: B terms, term scales, partial regions
  const size_t b_bytes = ncols * k, ts_off = (b_bytes + 255) / 256 * 256, part_off = ts_off + 256;
  const size_t need = part_off + (split > 1 ? split * m * n * 4 : 0);
  unsigned char* scratch = stream_scratch(st, need);
  if (scratch == nullptr) return kUnsupportedFeature;
  float* term_scale = reinterpret_cast<float*>(scratch + ts_off);
  float* part = reinterpret_cast<float*>(scratch + part_off);
  CUtensorMap wmap, bmap;
  if (int rc = byte_matrix_map(w, n, k, kTileM, &wmap)) return rc;
  if (int rc = byte_matrix_map(scratch, ncols, k, static_cast<uint32_t>(ncols), &bmap)) return rc;
  const unsigned pad_cols = static_cast<unsigned>(ncols - m * kTerms);
  const bool pdl_terms = pdl_allowed(st, nullptr, 0, scratch, need);
  launch_kernel(activation_terms_kernel, dim3(static_cast<unsigned>(m) + pad_cols, static_cast<unsigned>((k + kTermChunk - 1) / kTermChunk)),
                dim3(256), 0, st, pdl_terms, a, scratch, term_scale, static_cast<int>(m), static_cast<int>(k),
                static_cast<int>(ncols));
  if (int rc = check_launch()) return rc;
  F8Params p{scale, term_scale, split > 1 ? part : c, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
             static_cast<int>(ncols), static_cast<int>(stages_per_cta), static_cast<int>(total_stages), ring, 1};
  const size_t smem = 1024 + static_cast<size_t>(ring) * stage_bytes + 256;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&gemm_f8_umma_kernel), 227 * 1024)) return rc;
  // before its wait the tile kernel reads weights only; the kernel ahead of it (the terms) writes scratch
  pdl_allowed(st, nullptr, 0, split > 1 ? static_cast<void*>(part) : static_cast<void*>(c), m * n * 4);
  launch_kernel(gemm_f8_umma_kernel, dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(split)), dim3(kThreads),
                smem, st, true, wmap, bmap, p);
  if (int rc = check_launch()) return rc;
  if (split > 1) return tsr_gemm_vec_reduce(part, c, m * n, split, st);
  return kOk;
}

int umma_f8_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_f8_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}
int umma_f8_set_error_word(unsigned int* word) { return set_host_error_word(word); }

}  // namespace tsr
