// tcgen05 / TMEM tiles for the small-batch projections (m >= 9: the
// speculative-verify and chunked-prefill shapes, ids gemm_*_batched,
// gemm_*_wmma, gemm_mxfp4_rows/_batched, gemm_fp8).
//
// C[m,n] = A[m,k] . dq(W[n,k])^T with the roles swapped for the tensor core:
// the 128 weight rows of a CTA are the M side of tcgen05.mma (kind::f16, fp32
// accumulate in TMEM), the tokens are the N side.  Each fp32 activation is
// split into two fp16 columns (hi = fp16(a), lo = fp16(a - hi)), so the
// activation keeps ~22 bits; weights are dequantised to fp16 exactly as the
// reference's own tensor-core tile does (src/backends/rocm/rocm_kernels_wmma.cpp:
// 54-80 of the reference: weights dequantised to fp16 in shared memory).
//
// Per CTA: four producer warps (thread = weight row, and = one operand-B row)
// dequantise a 64-wide k slab into the canonical K-major no-swizzle UMMA
// layout (8x16-byte core matrices; leading-byte offset 128 B along k, stride
// byte offset 1024 B along rows), fence it to the async proxy and signal a
// full barrier; one elected thread issues four K=16 MMAs per slab and commits
// them to the slab's empty barrier; two slab buffers overlap dequantisation
// with the MMAs.  The producer warps then read the accumulator with tcgen05.ld
// (warp w owns TMEM lanes 32*(w%4)..), add the hi and lo columns and store C.
// Every wait is bounded and TMEM is always released.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "codec.cuh"
#include "launch.h"
#include "pipeline.cuh"

namespace tsr {

__device__ unsigned int g_umma_timeouts = 0;

namespace {

constexpr int kTileM = 128;       // weight rows per CTA
constexpr int kSlab = 64;         // k elements per pipeline step
constexpr int kMaxTokens = 64;    // tokens per CTA (N = 2 * padded tokens <= 128)
constexpr int kProducerThreads = 128;
constexpr int kUmmaThreads = kProducerThreads + 32;
constexpr int kASlabBytes = kTileM * kSlab * 2;  // 16384
constexpr uint32_t kLbo = 128, kSbo = (kSlab / 8) * 128;  // bytes

enum Format { kFmtQ4K = 0, kFmtQ6K = 1, kFmtMxFp4 = 2, kFmtFp8 = 3 };

struct UmmaParams {
  const float* a;
  const unsigned char* w;
  const float* scale;  // FP8 row scales
  float* c;
  int m, n, k;
};

// ---- tcgen05 wrappers -------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{.reg .pred p; setp.ne.b32 p, %4, 0; "
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major, no swizzle (layout type 0), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((kLbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((kSbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  return d;
}

// kind::f16: D fp32, A and B fp16, both K-major, M = 128, N = n_cols.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n_cols) {
  return (1u << 4) | ((n_cols >> 3) << 17) | ((kTileM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ---- per-format dequantisation of 64 consecutive weights of one row --------
// `slab` indexes 64-element pieces of the row; out[e] is weight k = 64*slab + e
// with the reference's arithmetic (src/core/numerics/quant.cpp:656-675,
// 421-449, 279-297; gemm.cpp:266-270).
template <int FMT>
__device__ __forceinline__ void dequant64(const UmmaParams& p, int row, int slab, float (&out)[64]) {
  if (FMT == kFmtQ4K) {
    const int nb = p.k / 256, b = slab >> 2, g = slab & 3;
    const unsigned char* blk = p.w + (static_cast<size_t>(row) * nb + b) * kQ4KBlockBytes;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * g));
    const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(blk + 32 + 32 * g));
    const float d = fp16_bits_to_float(hdr.x & 0xFFFFu), dmin = fp16_bits_to_float(hdr.x >> 16);
    const uint32_t s[3] = {hdr.y, hdr.z, hdr.w};
    uint32_t sc0, mn0, sc1, mn1;
    q4k_scale_min(s, 2 * g, sc0, mn0);
    q4k_scale_min(s, 2 * g + 1, sc1, mn1);
    const float dl = d * static_cast<float>(sc0), ml = dmin * static_cast<float>(mn0);
    const float dh = d * static_cast<float>(sc1), mh = dmin * static_cast<float>(mn1);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const uint32_t byte = (qw[e >> 2] >> (8 * (e & 3))) & 0xFFu;
      out[e] = fmaf(dl, static_cast<float>(byte & 15u), -ml);
      out[32 + e] = fmaf(dh, static_cast<float>(byte >> 4), -mh);
    }
  } else if (FMT == kFmtQ6K) {
    const int nb = p.k / 256, b = slab >> 2, j = slab & 3, h = j >> 1, hi = j & 1;
    const unsigned char* blk = p.w + (static_cast<size_t>(row) * nb + b) * kQ6KBlockBytes;
    const float d = fp16_bits_to_float(blk[208] | (blk[209] << 8));
    const unsigned char* ql = blk + 64 * h;
    const unsigned char* qh = blk + 128 + 32 * h;
    const signed char* sc = reinterpret_cast<const signed char*>(blk + 192 + 8 * h);
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      const int pp = 2 * hi + part;  // 0..3: which 32-element run of the half
#pragma unroll
      for (int l = 0; l < 32; ++l) {
        const uint32_t lo = ql[32 * (pp & 1) + l];
        const uint32_t nib = (pp & 2) ? (lo >> 4) : (lo & 15u);
        const int q = static_cast<int>(nib | (((static_cast<uint32_t>(qh[l]) >> (2 * pp)) & 3u) << 4)) - 32;
        out[32 * part + l] = d * static_cast<float>(sc[l / 16 + 2 * pp]) * static_cast<float>(q);
      }
    }
  } else if (FMT == kFmtMxFp4) {
    const unsigned char* nib = p.w + static_cast<size_t>(row) * (p.k / 2) + slab * 32;
    const unsigned char* scales = p.w + static_cast<size_t>(p.n) * (p.k / 2) + static_cast<size_t>(row) * (p.k / 32) + slab * 2;
    const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(nib));
    const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(nib + 16));
    const float s0 = e8m0_to_float(scales[0]), s1 = e8m0_to_float(scales[1]);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int e = 0; e < 64; ++e)
      out[e] = (e < 32 ? s0 : s1) * e2m1_to_float((qw[e >> 3] >> (4 * (e & 7))) & 15u);
  } else {
    const unsigned char* wr = p.w + static_cast<size_t>(row) * p.k + slab * 64;
    const float s = __ldg(p.scale + row);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(wr + 16 * v));
      const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 16; ++e) out[16 * v + e] = s * e4m3_to_float((qw[e >> 2] >> (8 * (e & 3))) & 0xFFu);
    }
  }
}

// Store 64 values of operand row `r` (k slab) into the canonical layout.
__device__ __forceinline__ void store_row_slab(unsigned char* tile, int r, const float (&v)[64]) {
  unsigned char* base = tile + (r >> 3) * kSbo + (r & 7) * 16;
#pragma unroll
  for (int kc = 0; kc < 8; ++kc) {
    uint4 u;
    u.x = pack_h2(v[8 * kc + 0], v[8 * kc + 1]);
    u.y = pack_h2(v[8 * kc + 2], v[8 * kc + 3]);
    u.z = pack_h2(v[8 * kc + 4], v[8 * kc + 5]);
    u.w = pack_h2(v[8 * kc + 6], v[8 * kc + 7]);
    *reinterpret_cast<uint4*>(base + kc * kLbo) = u;
  }
}

template <int FMT>
__global__ void __launch_bounds__(kUmmaThreads)
gemm_umma_kernel(const UmmaParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * kTileM;
  const int tok0 = blockIdx.y * kMaxTokens;
  const int tokens = min(kMaxTokens, p.m - tok0);
  const int tok_pad = (tokens + 7) & ~7;      // hi rows [0, tok_pad), lo rows [tok_pad, 2*tok_pad)
  const int n_cols = 2 * tok_pad;             // multiple of 16, <= 128
  const int b_slab_bytes = n_cols * kSlab * 2;
  unsigned char* a_tile[2] = {smem, smem + kASlabBytes};
  unsigned char* b_tile[2] = {smem + 2 * kASlabBytes, smem + 2 * kASlabBytes + b_slab_bytes};
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kASlabBytes + 2 * b_slab_bytes);
  uint64_t* full = bars;       // [2] producers -> MMA
  uint64_t* empty = bars + 2;  // [2] MMA -> producers
  uint64_t* done = bars + 4;   // accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(n_cols)) tmem_cols <<= 1;
  const int nslabs = p.k / kSlab;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&full[s], kProducerThreads);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, tmem_cols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool failed = false;

  if (warp < 4) {
    // ---------------- producers: dequantise A rows, convert B rows ---------
    const int wrow = row0 + tid;  // weight row of this thread
    for (int s = 0; s < nslabs && !failed; ++s) {
      const int buf = s & 1, round = s >> 1;
      if (round > 0 && !mbar_wait(&empty[buf], (round - 1) & 1, &g_umma_timeouts)) {
        failed = true;
        break;
      }
      float v[64];
      if (wrow < p.n) {
        dequant64<FMT>(p, wrow, s, v);
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) v[e] = 0.0f;
      }
      store_row_slab(a_tile[buf], tid, v);
      if (tid < n_cols) {
        const int tok = tid < tok_pad ? tid : tid - tok_pad;
        const bool lo_part = tid >= tok_pad;
        if (tok < tokens) {
          const float4* src = reinterpret_cast<const float4*>(p.a + static_cast<size_t>(tok0 + tok) * p.k + s * kSlab);
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const float4 x = __ldg(src + q);
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float cx = fminf(fmaxf(xs[e], -65504.0f), 65504.0f);
              const float hi = __half2float(__float2half_rn(cx));
              v[4 * q + e] = lo_part ? fminf(fmaxf(xs[e] - hi, -65504.0f), 65504.0f) : cx;
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; ++e) v[e] = 0.0f;
        }
        store_row_slab(b_tile[buf], tid, v);
      }
      fence_async_proxy();
      mbar_arrive(&full[buf]);
    }
  } else if (lane == 0) {
    // ---------------- MMA issuer --------------------------------------------
    const uint32_t idesc = instr_desc(static_cast<uint32_t>(n_cols));
    for (int s = 0; s < nslabs; ++s) {
      const int buf = s & 1, round = s >> 1;
      if (!mbar_wait(&full[buf], round & 1, &g_umma_timeouts)) {
        failed = true;
        break;
      }
      tcgen05_fence_after();
      const uint32_t a_addr = smem_u32(a_tile[buf]), b_addr = smem_u32(b_tile[buf]);
#pragma unroll
      for (int kk = 0; kk < kSlab / 16; ++kk) {
        umma_f16(tmem_base, smem_desc(a_addr + kk * 2 * kLbo), smem_desc(b_addr + kk * 2 * kLbo), idesc,
                 (s > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(&empty[buf]);  // the slab buffer is free once these MMAs have read it
    }
    umma_commit(done);
  }

  // ---------------- epilogue: TMEM -> registers -> C ------------------------
  if (warp < 4) {
    // warp-uniform, so the aligned TMEM loads below are never reached by part of a warp
    const bool ok = __all_sync(0xFFFFFFFFu, !failed && mbar_wait(done, 0, &g_umma_timeouts));
    tcgen05_fence_after();
    if (ok) {
      const int out_row = row0 + tid;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      for (int c0 = 0; c0 < tok_pad; c0 += 8) {
        float hi[8], lo[8];
        tmem_ld8(lane_addr + c0, hi);
        tmem_ld8(lane_addr + tok_pad + c0, lo);
        if (out_row < p.n) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c0 + j < tokens) p.c[static_cast<size_t>(tok0 + c0 + j) * p.n + out_row] = hi[j] + lo[j];
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, tmem_cols);
}

template <int FMT>
int launch_umma(const UmmaParams& p, cudaStream_t st) {
  const int tok_pad = ((p.m < kMaxTokens ? p.m : kMaxTokens) + 7) & ~7;
  const size_t smem = 2 * kASlabBytes + 2 * static_cast<size_t>(2 * tok_pad) * kSlab * 2 + 64 + 1024;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gemm_umma_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    attr = true;
  }
  const dim3 grid(static_cast<unsigned>((p.n + kTileM - 1) / kTileM),
                  static_cast<unsigned>((p.m + kMaxTokens - 1) / kMaxTokens));
  gemm_umma_kernel<FMT><<<grid, kUmmaThreads, smem, st>>>(p);
  return check_launch();
}

}  // namespace

// fmt: 0 Q4_K, 1 Q6_K, 2 MXFP4 (packed blob||scales), 3 FP8 (+ row scales).
// Returns kUnsupportedFeature when the shape is outside the tile's range.
int umma_gemm(int fmt, const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n,
              uint64_t k, cudaStream_t st) {
  if (k % kSlab != 0 || (fmt <= 1 && k % 256 != 0)) return kUnsupportedFeature;
  const UmmaParams p{a, static_cast<const unsigned char*>(w), scale, c, static_cast<int>(m),
                     static_cast<int>(n), static_cast<int>(k)};
  switch (fmt) {
    case kFmtQ4K: return launch_umma<kFmtQ4K>(p, st);
    case kFmtQ6K: return launch_umma<kFmtQ6K>(p, st);
    case kFmtMxFp4: return launch_umma<kFmtMxFp4>(p, st);
    case kFmtFp8: return launch_umma<kFmtFp8>(p, st);
    default: return kInvalidArgument;
  }
}

int umma_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_umma_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}

}  // namespace tsr
