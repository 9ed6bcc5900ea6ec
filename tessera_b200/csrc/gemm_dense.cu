// Projections over unquantised weights: ids "gemm_f32", "gemm_f32_batched" (fp32 weights: router gates, small
// heads) and "gemm_bf16", "gemm_bf16_batched", "gemm_bf16_wmma", "gemm_bf16_rows" (bf16 checkpoints).
// Contract: buffers A (fp32, m x k), W (n x k, fp32 or bf16), C (fp32, m x n); scalars m, n, k
// (include/tessera/backend.hpp:180-190 of the reference); arithmetic: GemmF32Ref, GemmBf16Ref
// (src/core/numerics/gemm.cpp:205-252): fp32 multiply-adds of a[i][t] and the weight widened to fp32.
//
// HBM-bound on W for the few rows of a decode or verify step: one warp per weight row, its lanes stride
// over k in 16-byte pieces (a row is read as contiguous 512-byte lines), up to eight activation rows are
// served from one pass over the weight row (the activations come from L1 / L2), partial sums meet by
// shuffles.  More than eight rows take further passes over the same weight row, which is then in L2.
// Three shapes of the same loop: a warp per weight row (one activation row over many weight rows), a CTA per
// weight row (few weight rows), four weight rows per warp (batches).
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"
#include "tessera_b200.h"

namespace tsr {
namespace {

constexpr int kDenseWarps = 8, kDenseRows = 8;

template <bool BF16>
__device__ __forceinline__ void widen(const uint4& raw, float (&w)[BF16 ? 8 : 4]) {
  if constexpr (BF16) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[2 * i] = __uint_as_float(words[i] << 16);
      w[2 * i + 1] = __uint_as_float(words[i] & 0xFFFF0000u);
    }
  } else {
    w[0] = __uint_as_float(raw.x), w[1] = __uint_as_float(raw.y), w[2] = __uint_as_float(raw.z), w[3] = __uint_as_float(raw.w);
  }
}

template <bool BF16>
__device__ __forceinline__ float weight_at(const void* w, size_t idx) {
  if constexpr (BF16) return __uint_as_float(static_cast<uint32_t>(static_cast<const unsigned short*>(w)[idx]) << 16);
  else return static_cast<const float*>(w)[idx];
}

// VEC: rows of W start on 16-byte boundaries and k is a multiple of the piece (k % 4 == 0 for fp32, % 8 for bf16).
// ROWS activation rows per pass (the last pass of a ragged batch repeats its last row and drops the copies).
// WPR warps share a weight row (its pieces dealt round-robin, the partial sums meet in shared memory): 8 when
// there are few weight rows, so that a small projection still fills the machine, else 1.
template <bool BF16, bool VEC, int ROWS, int WPR>
__global__ void __launch_bounds__(kDenseWarps * 32)
gemm_dense_kernel(const float* __restrict__ a, const void* __restrict__ w, float* __restrict__ c, int m, int n, int k) {
  constexpr int PIECE = BF16 ? 8 : 4, BATCH = 4;  // weight pieces a lane has in flight
  __shared__ float meet[kDenseWarps][ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j = blockIdx.x * (kDenseWarps / WPR) + warp / WPR, share = warp % WPR;
  const bool live = j < n;
  for (int i0 = 0; i0 < m; i0 += ROWS) {
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.0f;
    if (live) {
      if constexpr (VEC) {
        const uint4* wrow = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(w) +
                                                           static_cast<size_t>(j) * k * (BF16 ? 2 : 4));
        const int pieces = k / PIECE, stride = 32 * WPR;
        for (int t0 = share * 32 + lane; t0 < pieces; t0 += BATCH * stride) {
          uint4 raw[BATCH];
#pragma unroll
          for (int u = 0; u < BATCH; ++u)
            if (t0 + u * stride < pieces) raw[u] = __ldg(wrow + t0 + u * stride);
#pragma unroll
          for (int u = 0; u < BATCH; ++u) {
            const int t = t0 + u * stride;
            if (t < pieces) {
              float wf[PIECE];
              widen<BF16>(raw[u], wf);
#pragma unroll
              for (int r = 0; r < ROWS; ++r) {
                const float4* ar = reinterpret_cast<const float4*>(a + static_cast<size_t>(min(i0 + r, m - 1)) * k + t * PIECE);
#pragma unroll
                for (int q = 0; q < PIECE / 4; ++q) {
                  const float4 x = __ldg(ar + q);
                  acc[r] = fmaf(x.x, wf[4 * q], acc[r]);
                  acc[r] = fmaf(x.y, wf[4 * q + 1], acc[r]);
                  acc[r] = fmaf(x.z, wf[4 * q + 2], acc[r]);
                  acc[r] = fmaf(x.w, wf[4 * q + 3], acc[r]);
                }
              }
            }
          }
        }
      } else {
        for (int t = share * 32 + lane; t < k; t += 32 * WPR) {
          const float wf = weight_at<BF16>(w, static_cast<size_t>(j) * k + t);
#pragma unroll
          for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(a[static_cast<size_t>(min(i0 + r, m - 1)) * k + t], wf, acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], o);
    }
    if constexpr (WPR == 1) {
      if (live && lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
          if (i0 + r < m) c[static_cast<size_t>(i0 + r) * n + j] = acc[r];
      }
    } else {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) meet[warp][r] = acc[r];
      }
      __syncthreads();
      if (live && share == 0 && lane < ROWS && i0 + lane < m) {
        float total = meet[warp][lane];
#pragma unroll
        for (int o = 1; o < WPR; ++o) total += meet[warp + o][lane];
        c[static_cast<size_t>(i0 + lane) * n + j] = total;
      }
      __syncthreads();
    }
  }
}

// Batches over many weight rows: a warp takes four neighbouring weight rows and walks them together, so that the
// activation pieces it loads (ROWS rows from L1) serve four weight rows; with one weight row per warp a batch of
// four is bound by those L1 loads (measured 0.29 of the HBM peak at m = 4 over bf16 17408 x 5120).
template <bool BF16, int ROWS>
__global__ void __launch_bounds__(kDenseWarps * 32)
gemm_dense_blocked_kernel(const float* __restrict__ a, const void* __restrict__ w, float* __restrict__ c, int m, int n, int k) {
  constexpr int PIECE = BF16 ? 8 : 4, NR = 4;
  const int lane = threadIdx.x & 31;
  const int j0 = (blockIdx.x * kDenseWarps + (threadIdx.x >> 5)) * NR;
  if (j0 >= n) return;
  const size_t row_bytes = static_cast<size_t>(k) * (BF16 ? 2 : 4);
  const unsigned char* wbase = static_cast<const unsigned char*>(w);
  const int pieces = k / PIECE;
  for (int i0 = 0; i0 < m; i0 += ROWS) {
    float acc[NR][ROWS];
#pragma unroll
    for (int u = 0; u < NR; ++u)
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[u][r] = 0.0f;
    for (int t = lane; t < pieces; t += 32) {
      uint4 raw[NR];
#pragma unroll
      for (int u = 0; u < NR; ++u)
        raw[u] = __ldg(reinterpret_cast<const uint4*>(wbase + static_cast<size_t>(min(j0 + u, n - 1)) * row_bytes) + t);
      float4 x[ROWS][PIECE / 4];
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int q = 0; q < PIECE / 4; ++q)
          x[r][q] = __ldg(reinterpret_cast<const float4*>(a + static_cast<size_t>(min(i0 + r, m - 1)) * k + t * PIECE) + q);
#pragma unroll
      for (int u = 0; u < NR; ++u) {
        float wf[PIECE];
        widen<BF16>(raw[u], wf);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
          for (int q = 0; q < PIECE / 4; ++q) {
            acc[u][r] = fmaf(x[r][q].x, wf[4 * q], acc[u][r]);
            acc[u][r] = fmaf(x[r][q].y, wf[4 * q + 1], acc[u][r]);
            acc[u][r] = fmaf(x[r][q].z, wf[4 * q + 2], acc[u][r]);
            acc[u][r] = fmaf(x[r][q].w, wf[4 * q + 3], acc[u][r]);
          }
      }
    }
#pragma unroll
    for (int u = 0; u < NR; ++u)
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        float v = acc[u][r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (lane == 0 && j0 + u < n && i0 + r < m) c[static_cast<size_t>(i0 + r) * n + j0 + u] = v;
      }
  }
}

template <bool BF16, bool VEC, int ROWS>
int launch_dense_rows(const float* a, const void* w, float* c, int m, int n, int k, cudaStream_t st) {
  if (n <= 2048) {  // few weight rows: a CTA per row
    gemm_dense_kernel<BF16, VEC, ROWS, kDenseWarps><<<static_cast<unsigned>(n), kDenseWarps * 32, 0, st>>>(a, w, c, m, n, k);
  } else if (VEC && ROWS > 1) {
    const unsigned grid = static_cast<unsigned>((n + kDenseWarps * 4 - 1) / (kDenseWarps * 4));
    gemm_dense_blocked_kernel<BF16, ROWS><<<grid, kDenseWarps * 32, 0, st>>>(a, w, c, m, n, k);
  } else {
    const unsigned grid = static_cast<unsigned>((n + kDenseWarps - 1) / kDenseWarps);
    gemm_dense_kernel<BF16, VEC, ROWS, 1><<<grid, kDenseWarps * 32, 0, st>>>(a, w, c, m, n, k);
  }
  return check_launch();
}

template <bool BF16, bool VEC>
int launch_dense(const float* a, const void* w, float* c, int m, int n, int k, cudaStream_t st) {
  if (m == 1) return launch_dense_rows<BF16, VEC, 1>(a, w, c, m, n, k, st);
  if (m == 2) return launch_dense_rows<BF16, VEC, 2>(a, w, c, m, n, k, st);
  if (m <= 4) return launch_dense_rows<BF16, VEC, 4>(a, w, c, m, n, k, st);
  return launch_dense_rows<BF16, VEC, kDenseRows>(a, w, c, m, n, k, st);
}

}  // namespace
}  // namespace tsr

using namespace tsr;

extern "C" int tsr_gemm_dense(int bf16, const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                              void* stream) {
  if (!a || !w || !c || m == 0 || n == 0 || k == 0 || m > 0x7FFFFFFFull || n > 0x7FFFFFFFull || k > 0x7FFFFFFFull)
    return kInvalidArgument;
  auto st = static_cast<cudaStream_t>(stream);
  const bool vec = k % (bf16 ? 8 : 4) == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0;
  const int mi = static_cast<int>(m), ni = static_cast<int>(n), ki = static_cast<int>(k);
  if (bf16) return vec ? launch_dense<true, true>(a, w, c, mi, ni, ki, st) : launch_dense<true, false>(a, w, c, mi, ni, ki, st);
  return vec ? launch_dense<false, true>(a, w, c, mi, ni, ki, st) : launch_dense<false, false>(a, w, c, mi, ni, ki, st);
}
