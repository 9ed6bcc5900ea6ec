// Warp-per-weight-row GEMV family on CUDA cores: the general path that
// serves every (m, n, k, split) the contracts allow, for all four weight
// formats.  One warp owns one weight row and up to MR activation rows, so a
// weight byte is read once per MR rows.  The bandwidth-critical shapes are
// taken over by the staged tensor-pipe kernels (gemv_mma.cu); this file is
// what runs for ragged shapes (k not a multiple of the staged tile, odd
// alignments) and is the simplest statement of each format's arithmetic.
//
// Arithmetic: fp32 throughout.  For the block formats the per-sub-block
// scale is applied to the sub-block's partial dot (d*sc*sum(q*a) -
// dmin*mn*sum(a)), which is the reference sum re-associated.
#include "codec.cuh"
#include "launch.h"

namespace tsr {

constexpr int kWarpsPerBlock = 8;

// ---------------------------------------------------------------- Q4_K
// Lane (sub = lane/8, c = lane%8): block b0+sub+4*it, 16-byte chunk c of the
// 128 nibble bytes: group g = c/2, low nibbles -> elements 64g+16(c&1)+e,
// high nibbles -> +32 (src/core/numerics/quant.cpp:656-675).
template <int MR>
__global__ void __launch_bounds__(256)
gemv_q4k_rows_kernel(const float* __restrict__ a, const uint8_t* __restrict__ w,
                     float* __restrict__ c, int mrows, int n, int k, int split,
                     size_t region_stride) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const int nb = k / kBlockElems;
  const int per = nb / split;
  const int b0 = blockIdx.y * per;
  const uint8_t* wrow = w + static_cast<size_t>(row) * nb * kQ4KBlockBytes;
  const int sub = lane >> 3, c8 = lane & 7, g = c8 >> 1, half = c8 & 1;
  float acc[MR];
#pragma unroll
  for (int i = 0; i < MR; ++i) acc[i] = 0.0f;
  for (int b = b0 + sub; b < b0 + per; b += 4) {
    const uint8_t* blk = wrow + static_cast<size_t>(b) * kQ4KBlockBytes;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(blk + 16 + c8 * 16));
    const float d = fp16_bits_to_float(hdr.x & 0xFFFFu);
    const float dmin = fp16_bits_to_float(hdr.x >> 16);
    const uint32_t s[3] = {hdr.y, hdr.z, hdr.w};
    uint32_t sc0, mn0, sc1, mn1;
    q4k_scale_min(s, 2 * g, sc0, mn0);
    q4k_scale_min(s, 2 * g + 1, sc1, mn1);
    const float dl = d * static_cast<float>(sc0), ml = dmin * static_cast<float>(mn0);
    const float dh = d * static_cast<float>(sc1), mh = dmin * static_cast<float>(mn1);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    const int kbase = b * kBlockElems + g * 64 + half * 16;
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      if (i < mrows) {
        const float4* alo = reinterpret_cast<const float4*>(a + static_cast<size_t>(i) * k + kbase);
        const float4* ahi = alo + 8;
        float sql = 0.f, sl = 0.f, sqh = 0.f, sh = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 x = __ldg(alo + v), y = __ldg(ahi + v);
          const uint32_t word = qw[v];
          const float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t byte = (word >> (8 * e)) & 0xFFu;
            sql = fmaf(static_cast<float>(byte & 15u), xs[e], sql);
            sqh = fmaf(static_cast<float>(byte >> 4), ys[e], sqh);
            sl += xs[e];
            sh += ys[e];
          }
        }
        acc[i] += dl * sql - ml * sl + dh * sqh - mh * sh;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const float sum = warp_sum(acc[i]);
    if (lane == 0 && i < mrows)
      c[blockIdx.y * region_stride + static_cast<size_t>(i) * n + row] = sum;
  }
}

// ---------------------------------------------------------------- Q6_K
// 210-byte blocks are only 2-byte aligned, so this path reads 16-bit words.
// Lane (h = lane/16, j = lane%16) of a block takes ql[64h+2j..], ql[64h+32+2j..]
// and qh[32h+2j..]: two adjacent positions of each of the four 32-element runs
// of half h, i.e. elements 128h + 32*run + 2j + {0,1}
// (src/core/numerics/quant.cpp:421-449).  Integers become floats through the
// 2^23 magic constant instead of conversion instructions.
template <int MR>
__global__ void __launch_bounds__(256)
gemv_q6k_rows_kernel(const float* __restrict__ a, const uint8_t* __restrict__ w,
                     float* __restrict__ c, int mrows, int n, int k, int split,
                     size_t region_stride) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const int nb = k / kBlockElems;
  const int per = nb / split;
  const int b0 = blockIdx.y * per;
  const uint8_t* wrow = w + static_cast<size_t>(row) * nb * kQ6KBlockBytes;
  const int h = lane >> 4, j = lane & 15;
  constexpr float kMagic = 8388608.0f + 32.0f;  // (q | 0x4B000000) - kMagic = q - 32
  float acc[MR];
#pragma unroll
  for (int i = 0; i < MR; ++i) acc[i] = 0.0f;
#pragma unroll 4
  for (int b = b0; b < b0 + per; ++b) {
    const unsigned short* blk = reinterpret_cast<const unsigned short*>(wrow + static_cast<size_t>(b) * kQ6KBlockBytes);
    const uint32_t l0 = __ldg(blk + 32 * h + j);        // ql[64h + 2j, +1]
    const uint32_t l1 = __ldg(blk + 32 * h + 16 + j);   // ql[64h + 32 + 2j, +1]
    const uint32_t qh = __ldg(blk + 64 + 16 * h + j);   // qh[32h + 2j, +1]
    const float d = fp16_bits_to_float(__ldg(blk + 104));
    // scales of half h: bytes 192 + 8h .. +7; run r of this lane uses byte (j>>3) + 2r
    const uint32_t s01 = __ldg(blk + 96 + 4 * h + 0), s23 = __ldg(blk + 96 + 4 * h + 1);
    const uint32_t s45 = __ldg(blk + 96 + 4 * h + 2), s67 = __ldg(blk + 96 + 4 * h + 3);
    const int sh = 8 * (j >> 3);
    const float sc[4] = {static_cast<float>(static_cast<signed char>((s01 >> sh) & 0xFF)),
                         static_cast<float>(static_cast<signed char>((s23 >> sh) & 0xFF)),
                         static_cast<float>(static_cast<signed char>((s45 >> sh) & 0xFF)),
                         static_cast<float>(static_cast<signed char>((s67 >> sh) & 0xFF))};
    // runs: 0 = low nibble of l0, 1 = low nibble of l1, 2 = high nibble of l0, 3 = high nibble of l1
    float wv[4][2];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t lw = (r & 1) ? l1 : l0;
      const uint32_t nib = (r & 2) ? (lw >> 4) : lw;
      const uint32_t hi2 = qh >> (2 * r);
      const uint32_t q0 = (nib & 0xFu) | ((hi2 & 3u) << 4);
      const uint32_t q1 = ((nib >> 8) & 0xFu) | (((hi2 >> 8) & 3u) << 4);
      const float ds = d * sc[r];
      wv[r][0] = ds * (__uint_as_float(q0 | 0x4B000000u) - kMagic);
      wv[r][1] = ds * (__uint_as_float(q1 | 0x4B000000u) - kMagic);
    }
    const int kbase = b * kBlockElems + 128 * h + 2 * j;
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      if (i < mrows) {
        const float* ar = a + static_cast<size_t>(i) * k + kbase;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float2 x = __ldg(reinterpret_cast<const float2*>(ar + 32 * r));
          acc[i] = fmaf(x.x, wv[r][0], acc[i]);
          acc[i] = fmaf(x.y, wv[r][1], acc[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const float sum = warp_sum(acc[i]);
    if (lane == 0 && i < mrows)
      c[blockIdx.y * region_stride + static_cast<size_t>(i) * n + row] = sum;
  }
}

// ---------------------------------------------------------------- MXFP4
// Lane l takes 32-element blocks l, l+32, ... of the row: 16 nibble bytes
// plus one E8M0 byte (src/core/numerics/gemm.cpp:311-344; low nibble is the
// even element).
template <int MR>
__global__ void __launch_bounds__(256)
gemv_mxfp4_rows_kernel(const float* __restrict__ a, const uint8_t* __restrict__ w,
                       float* __restrict__ c, int mrows, int n, int k) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const int nb = k / 32;
  const uint8_t* nib = w + static_cast<size_t>(row) * (k / 2);
  const uint8_t* scales = w + static_cast<size_t>(n) * (k / 2) + static_cast<size_t>(row) * nb;
  float acc[MR];
#pragma unroll
  for (int i = 0; i < MR; ++i) acc[i] = 0.0f;
  for (int b = lane; b < nb; b += 32) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(nib + static_cast<size_t>(b) * 16));
    const float scale = e8m0_to_float(__ldg(scales + b));
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    float wv[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) wv[e] = e2m1_to_float((qw[e >> 3] >> (4 * (e & 7))) & 15u);
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      if (i < mrows) {
        const float4* ar = reinterpret_cast<const float4*>(a + static_cast<size_t>(i) * k + b * 32);
        float part = 0.f;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const float4 x = __ldg(ar + v);
          part = fmaf(x.x, wv[4 * v + 0], part);
          part = fmaf(x.y, wv[4 * v + 1], part);
          part = fmaf(x.z, wv[4 * v + 2], part);
          part = fmaf(x.w, wv[4 * v + 3], part);
        }
        acc[i] = fmaf(scale, part, acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const float sum = warp_sum(acc[i]);
    if (lane == 0 && i < mrows) c[static_cast<size_t>(i) * n + row] = sum;
  }
}

// ---------------------------------------------------------------- FP8
// Lane takes 16 weight bytes per step; weight = s[row] * e4m3
// (src/core/numerics/gemm.cpp:253-277), the row scale applied to the dot.
template <int MR>
__global__ void __launch_bounds__(256)
gemv_fp8_rows_kernel(const float* __restrict__ a, const uint8_t* __restrict__ w,
                     const float* __restrict__ s, float* __restrict__ c, int mrows, int n, int k) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const uint8_t* wrow = w + static_cast<size_t>(row) * k;
  float acc[MR];
#pragma unroll
  for (int i = 0; i < MR; ++i) acc[i] = 0.0f;
  const bool vec = (k % 16 == 0);
  if (vec) {
    for (int t = lane * 16; t < k; t += 32 * 16) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(wrow + t));
      const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
      float wv[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) wv[e] = e4m3_to_float((qw[e >> 2] >> (8 * (e & 3))) & 0xFFu);
#pragma unroll
      for (int i = 0; i < MR; ++i) {
        if (i < mrows) {
          const float4* ar = reinterpret_cast<const float4*>(a + static_cast<size_t>(i) * k + t);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const float4 x = __ldg(ar + v);
            acc[i] = fmaf(x.x, wv[4 * v + 0], acc[i]);
            acc[i] = fmaf(x.y, wv[4 * v + 1], acc[i]);
            acc[i] = fmaf(x.z, wv[4 * v + 2], acc[i]);
            acc[i] = fmaf(x.w, wv[4 * v + 3], acc[i]);
          }
        }
      }
    }
  } else {
    for (int t = lane; t < k; t += 32) {
      const float wv = e4m3_to_float(__ldg(wrow + t));
#pragma unroll
      for (int i = 0; i < MR; ++i)
        if (i < mrows) acc[i] = fmaf(__ldg(a + static_cast<size_t>(i) * k + t), wv, acc[i]);
    }
  }
  const float scale = __ldg(s + row);
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const float sum = warp_sum(acc[i]);
    if (lane == 0 && i < mrows) c[static_cast<size_t>(i) * n + row] = sum * scale;
  }
}

// ---------------------------------------------------------------- W4A8
// "gemm_mxfp4_wmma" contract on CUDA cores
// (src/backends/vulkan/kernels/gemm_mxfp4_wmma.comp:78-117): the weight
// nibble is folded to an E4M3 byte relative to the row's largest block
// scale, multiplied with the E4M3 activation code, and the sum is scaled by
// As[r] * 2^(wref-127).  Region y of C covers 128-element chunks
// [y*per, (y+1)*per).
template <int MR>
__global__ void __launch_bounds__(256)
gemv_w4a8_rows_kernel(const uint8_t* __restrict__ a8, const uint8_t* __restrict__ w,
                      const float* __restrict__ as, const uint8_t* __restrict__ wref,
                      float* __restrict__ c, int mrows, int n, int k, int split,
                      size_t region_stride) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const int nb = k / 32;
  const int chunks = (k + 127) / 128;
  const int per = (chunks + split - 1) / split;
  int k_lo = blockIdx.y * per * 128;
  int k_hi = min(k_lo + per * 128, k);
  k_lo = min(k_lo, k);
  const uint8_t* nib = w + static_cast<size_t>(row) * (k / 2);
  const uint8_t* scales = w + static_cast<size_t>(n) * (k / 2) + static_cast<size_t>(row) * nb;
  const uint32_t ref = __ldg(wref + row);
  float acc[MR];
#pragma unroll
  for (int i = 0; i < MR; ++i) acc[i] = 0.0f;
  for (int b = k_lo / 32 + lane; b < k_hi / 32; b += 32) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(nib + static_cast<size_t>(b) * 16));
    int d = static_cast<int>(ref) - static_cast<int>(__ldg(scales + b));
    d = max(0, min(15, d));
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    float wv[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const uint32_t v = (qw[e >> 3] >> (4 * (e & 7))) & 15u;
      wv[e] = e4m3_to_float(fold_code(static_cast<uint32_t>(d), v & 7u) | ((v & 8u) << 4));
    }
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      if (i < mrows) {
        const uint4* ar = reinterpret_cast<const uint4*>(a8 + static_cast<size_t>(i) * k + b * 32);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const uint4 x = __ldg(ar + v);
          const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int e = 0; e < 16; ++e)
            acc[i] = fmaf(e4m3_to_float((xw[e >> 2] >> (8 * (e & 3))) & 0xFFu), wv[16 * v + e],
                          acc[i]);
        }
      }
    }
  }
  const float wscale = e8m0_to_float(ref);
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const float sum = warp_sum(acc[i]);
    if (lane == 0 && i < mrows)
      c[blockIdx.y * region_stride + static_cast<size_t>(i) * n + row] =
          sum * __ldg(as + i) * wscale;
  }
}

// ------------------------------------------------------------- launchers

template <typename F>
static int for_row_chunks(uint64_t m, F&& launch_chunk) {
  for (uint64_t i0 = 0; i0 < m; i0 += 8) {
    const int rows = static_cast<int>(m - i0 < 8 ? m - i0 : 8);
    launch_chunk(i0, rows);
  }
  return check_launch();
}

#define TSR_DISPATCH_MR(rows, CALL) \
  do {                              \
    if ((rows) == 1) {              \
      CALL(1);                      \
    } else if ((rows) == 2) {       \
      CALL(2);                      \
    } else if ((rows) <= 4) {       \
      CALL(4);                      \
    } else {                        \
      CALL(8);                      \
    }                               \
  } while (0)

int rows_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                  uint64_t split, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(split));
  return for_row_chunks(m, [&](uint64_t i0, int rows) {
#define CALL(MR)                                                                               \
  gemv_q4k_rows_kernel<MR><<<grid, 256, 0, st>>>(a + i0 * k, static_cast<const uint8_t*>(w),  \
                                                 c + i0 * n, rows, (int)n, (int)k, (int)split, \
                                                 m * n)
    TSR_DISPATCH_MR(rows, CALL);
#undef CALL
  });
}

int rows_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                  uint64_t split, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(split));
  return for_row_chunks(m, [&](uint64_t i0, int rows) {
#define CALL(MR)                                                                               \
  gemv_q6k_rows_kernel<MR><<<grid, 256, 0, st>>>(a + i0 * k, static_cast<const uint8_t*>(w),  \
                                                 c + i0 * n, rows, (int)n, (int)k, (int)split, \
                                                 m * n)
    TSR_DISPATCH_MR(rows, CALL);
#undef CALL
  });
}

int rows_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                    cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8));
  return for_row_chunks(m, [&](uint64_t i0, int rows) {
#define CALL(MR)                                                                                \
  gemv_mxfp4_rows_kernel<MR><<<grid, 256, 0, st>>>(a + i0 * k, static_cast<const uint8_t*>(w), \
                                                   c + i0 * n, rows, (int)n, (int)k)
    TSR_DISPATCH_MR(rows, CALL);
#undef CALL
  });
}

int rows_gemm_fp8(const float* a, const void* w, const float* s, float* c, uint64_t m, uint64_t n,
                  uint64_t k, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8));
  return for_row_chunks(m, [&](uint64_t i0, int rows) {
#define CALL(MR)                                                                              \
  gemv_fp8_rows_kernel<MR><<<grid, 256, 0, st>>>(a + i0 * k, static_cast<const uint8_t*>(w), \
                                                 s, c + i0 * n, rows, (int)n, (int)k)
    TSR_DISPATCH_MR(rows, CALL);
#undef CALL
  });
}

int rows_gemm_w4a8(const void* a8, const void* w, const float* as, const void* wref, float* c,
                   uint64_t m, uint64_t n, uint64_t k, uint64_t split, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(split));
  return for_row_chunks(m, [&](uint64_t i0, int rows) {
#define CALL(MR)                                                                         \
  gemv_w4a8_rows_kernel<MR><<<grid, 256, 0, st>>>(                                      \
      static_cast<const uint8_t*>(a8) + i0 * k, static_cast<const uint8_t*>(w), as + i0, \
      static_cast<const uint8_t*>(wref), c + i0 * n, rows, (int)n, (int)k, (int)split, m * n)
    TSR_DISPATCH_MR(rows, CALL);
#undef CALL
  });
}

}  // namespace tsr
