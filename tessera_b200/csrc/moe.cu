// Routed-expert kernels of a mixture-of-experts layer for one token: the expert
// ids live in device memory, so the launch gathers the rows of the selected
// experts out of the whole 3-D expert tensors.  Contracts:
// src/backends/rocm/rocm_kernels.hpp:604-640 of the reference (moe_gate,
// moe_scale_add, moe_experts_gate_up_q4k, moe_experts_down_q4k / _q6k); the
// arithmetic of a row is the reference's block dot
// (src/core/numerics/gemm.cpp:18-41,88-99), re-associated per sub-block as in
// the warp-per-row family (gemv_rows.cu).
//
// HBM-bound gathers: top_k experts x inter rows x (gate + up) and top_k x
// hidden rows per token (config 4: 9.4 MB + 4.7 MB per layer), every weight
// byte read once with 16-byte loads, the activations staged in shared memory.
#include "codec.cuh"
#include "launch.h"
#include "tessera_b200.h"

namespace tsr {

namespace {

constexpr int kMoeWarps = 8;

// What lane (c8 = lane % 8) contributes to the dot of one Q4_K block with 256 activations at
// `a`: 16-byte chunk c8 of the nibble bytes (group g = c8/2: low nibbles -> elements
// 64g + 16(c8&1) + e, high nibbles -> +32, src/core/numerics/quant.cpp:656-675), from the
// block's header and that chunk, both already loaded.
__device__ __forceinline__ float q4k_chunk_dot(const float* a, uint4 hdr, uint4 q, int c8) {
  const int g = c8 >> 1, half = c8 & 1;
  const float d = fp16_bits_to_float(hdr.x & 0xFFFFu);
  const float dmin = fp16_bits_to_float(hdr.x >> 16);
  const uint32_t s[3] = {hdr.y, hdr.z, hdr.w};
  uint32_t sc0, mn0, sc1, mn1;
  q4k_scale_min(s, 2 * g, sc0, mn0);
  q4k_scale_min(s, 2 * g + 1, sc1, mn1);
  const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
  const float4* alo = reinterpret_cast<const float4*>(a + g * 64 + half * 16);
  const float4* ahi = alo + 8;
  float sql = 0.f, sl = 0.f, sqh = 0.f, sh = 0.f;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const float4 x = alo[v], y = ahi[v];
    const float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t byte = (qw[v] >> (8 * e)) & 0xFFu;
      sql = fmaf(static_cast<float>(byte & 15u), xs[e], sql);
      sqh = fmaf(static_cast<float>(byte >> 4), ys[e], sqh);
      sl += xs[e];
      sh += ys[e];
    }
  }
  return d * static_cast<float>(sc0) * sql - dmin * static_cast<float>(mn0) * sl + d * static_cast<float>(sc1) * sqh -
         dmin * static_cast<float>(mn1) * sh;
}

// The same for one Q6_K block (210 bytes, 2-byte aligned): lane (h = lane/16, j = lane%16)
// takes elements 128h + 32r + 2j + {0,1}, r = 0..3 (src/core/numerics/quant.cpp:421-449).
__device__ __forceinline__ float q6k_block_share(const float* a, const uint8_t* block, int lane) {
  const int h = lane >> 4, j = lane & 15;
  constexpr float kMagic = 8388608.0f + 32.0f;  // (q | 0x4B000000) - kMagic = q - 32
  const unsigned short* blk = reinterpret_cast<const unsigned short*>(block);
  const uint32_t l0 = __ldg(blk + 32 * h + j), l1 = __ldg(blk + 32 * h + 16 + j), qh = __ldg(blk + 64 + 16 * h + j);
  const float d = fp16_bits_to_float(__ldg(blk + 104));
  const uint32_t s01 = __ldg(blk + 96 + 4 * h + 0), s23 = __ldg(blk + 96 + 4 * h + 1);
  const uint32_t s45 = __ldg(blk + 96 + 4 * h + 2), s67 = __ldg(blk + 96 + 4 * h + 3);
  const int sh = 8 * (j >> 3);
  const uint32_t sw[4] = {s01, s23, s45, s67};
  const float* ar = a + 128 * h + 2 * j;
  float acc = 0.0f;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t lw = (r & 1) ? l1 : l0;
    const uint32_t nib = (r & 2) ? (lw >> 4) : lw;
    const uint32_t hi2 = qh >> (2 * r);
    const uint32_t q0 = (nib & 0xFu) | ((hi2 & 3u) << 4);
    const uint32_t q1 = ((nib >> 8) & 0xFu) | (((hi2 >> 8) & 3u) << 4);
    const float ds = d * static_cast<float>(static_cast<signed char>((sw[r] >> sh) & 0xFF));
    const float2 x = *reinterpret_cast<const float2*>(ar + 32 * r);
    acc = fmaf(x.x, ds * (__uint_as_float(q0 | 0x4B000000u) - kMagic), acc);
    acc = fmaf(x.y, ds * (__uint_as_float(q1 | 0x4B000000u) - kMagic), acc);
  }
  return acc;
}

// phi[slot][j] = silu(G_e[j] . x) * (U_e[j] . x), e = ids[slot]: one warp per (slot, j), x in
// shared memory (dynamic: hidden floats).
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_gate_up_q4k_kernel(const float* __restrict__ x, const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                       const uint32_t* __restrict__ ids, float* __restrict__ phi, int hidden, int inter, int top_k,
                       size_t gate_stride, size_t up_stride, int experts) {
  extern __shared__ __align__(16) float xs[];
  for (int t = threadIdx.x; t < hidden / 4; t += blockDim.x)
    reinterpret_cast<float4*>(xs)[t] = __ldg(reinterpret_cast<const float4*>(x) + t);
  __syncthreads();
  const int idx = blockIdx.x * kMoeWarps + (threadIdx.x >> 5);
  if (idx >= inter * top_k) return;
  const int lane = threadIdx.x & 31;
  const int slot = idx / inter, j = idx - slot * inter;
  const uint32_t e = ids[slot];
  if (e >= static_cast<uint32_t>(experts)) {  // an id outside the tensors: write nothing wrong, read nothing wild
    if (lane == 0) phi[idx] = 0.0f;
    return;
  }
  const int nb = hidden / kBlockElems;
  const size_t row = static_cast<size_t>(j) * nb * kQ4KBlockBytes;
  const uint8_t* grow = gate + e * gate_stride + row;
  const uint8_t* urow = up + e * up_stride + row;
  // lane (sub = lane/8, c8 = lane%8): chunk c8 of blocks sub, sub + 4, ...; the loads of two
  // rounds of both rows are in flight before the first is used
  const int sub = lane >> 3, c8 = lane & 7;
  float g = 0.0f, u = 0.0f;
  for (int b0 = sub; b0 < nb; b0 += 8) {
    uint4 hg[2], qg[2], hu[2], qu[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int b = b0 + 4 * r;
      if (b < nb) {
        const uint8_t* gb = grow + static_cast<size_t>(b) * kQ4KBlockBytes;
        const uint8_t* ub = urow + static_cast<size_t>(b) * kQ4KBlockBytes;
        hg[r] = __ldg(reinterpret_cast<const uint4*>(gb));
        qg[r] = __ldg(reinterpret_cast<const uint4*>(gb + 16 + c8 * 16));
        hu[r] = __ldg(reinterpret_cast<const uint4*>(ub));
        qu[r] = __ldg(reinterpret_cast<const uint4*>(ub + 16 + c8 * 16));
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int b = b0 + 4 * r;
      if (b < nb) {
        g += q4k_chunk_dot(xs + b * kBlockElems, hg[r], qg[r], c8);
        u += q4k_chunk_dot(xs + b * kBlockElems, hu[r], qu[r], c8);
      }
    }
  }
  g = warp_sum(g);
  u = warp_sum(u);
  if (lane == 0) phi[idx] = (g / (1.0f + expf(-g))) * u;
}

// out[j] (+)= sum_slot wts[slot] * (D_e[j] . phi[slot]): one warp per j; phi (top_k x inter)
// in shared memory.
template <bool Q6>
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_down_kernel(const float* __restrict__ phi, const uint8_t* __restrict__ down, const uint32_t* __restrict__ ids,
                const float* __restrict__ wts, float* __restrict__ out, int hidden, int inter, int top_k,
                size_t down_stride, int accumulate, int experts) {
  extern __shared__ __align__(16) float ps[];
  for (int t = threadIdx.x; t < top_k * inter / 4; t += blockDim.x)
    reinterpret_cast<float4*>(ps)[t] = __ldg(reinterpret_cast<const float4*>(phi) + t);
  __syncthreads();
  const int j = blockIdx.x * kMoeWarps + (threadIdx.x >> 5);
  if (j >= hidden) return;
  const int lane = threadIdx.x & 31;
  const int nb = inter / kBlockElems;
  float acc = 0.0f;
  if (Q6) {
    // a whole warp per block; two (slot, block) pairs are loaded before the first is used
    for (int slot = 0; slot < top_k; ++slot) {
      const uint32_t e = ids[slot];
      if (e >= static_cast<uint32_t>(experts)) continue;
      const uint8_t* row = down + e * down_stride + static_cast<size_t>(j) * nb * kQ6KBlockBytes;
      float part = 0.0f;
#pragma unroll 2
      for (int b = 0; b < nb; ++b)
        part += q6k_block_share(ps + slot * inter + b * kBlockElems, row + static_cast<size_t>(b) * kQ6KBlockBytes, lane);
      acc = fmaf(wts[slot], part, acc);
    }
  } else {
    // the (slot, block) pairs of this output row, four at a time across the warp (lane/8) and
    // two such rounds in flight: the row of an expert is short (inter/256 blocks)
    const int sub = lane >> 3, c8 = lane & 7, pairs = top_k * nb;
    for (int p0 = sub; p0 < pairs; p0 += 8) {
      uint4 h[2], q[2];
      float w[2];
      int at[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int pr = p0 + 4 * r;
        w[r] = 0.0f;
        at[r] = 0;
        h[r] = q[r] = make_uint4(0u, 0u, 0u, 0u);
        if (pr < pairs) {
          const int slot = pr / nb, b = pr - slot * nb;
          const uint32_t e = ids[slot];
          if (e < static_cast<uint32_t>(experts)) {
            const uint8_t* blk = down + e * down_stride + (static_cast<size_t>(j) * nb + b) * kQ4KBlockBytes;
            h[r] = __ldg(reinterpret_cast<const uint4*>(blk));
            q[r] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + c8 * 16));
            w[r] = wts[slot];
            at[r] = slot * inter + b * kBlockElems;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) acc = fmaf(w[r], q4k_chunk_dot(ps + at[r], h[r], q[r], c8), acc);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[j] = accumulate ? out[j] + acc : acc;
}

// moe_gate: softmax over the top_k selected logits; sigmoid of the shared-expert gate x . w.
__global__ void __launch_bounds__(256)
moe_gate_kernel(const float* __restrict__ vals, const float* __restrict__ x, const float* __restrict__ w,
                float* __restrict__ wts, float* __restrict__ sig, int top_k, int hidden) {
  __shared__ float red[8];
  float dot = 0.0f;
  for (int t = threadIdx.x; t < hidden; t += blockDim.x) dot = fmaf(x[t], w[t], dot);
  dot = warp_sum(dot);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int i = 0; i < 8; ++i) total += red[i];
    float m = -3.402823466e+38f;
    for (int p = 0; p < top_k; ++p) m = fmaxf(m, vals[p]);
    float sum = 0.0f;
    for (int p = 0; p < top_k; ++p) sum += expf(vals[p] - m);
    for (int p = 0; p < top_k; ++p) wts[p] = expf(vals[p] - m) / sum;
    sig[0] = 1.0f / (1.0f + expf(-total));
  }
}

__global__ void moe_scale_add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                     const float* __restrict__ f, float* __restrict__ o, size_t n, size_t idx) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) o[i] = __fadd_rn(a[i], __fmul_rn(f[idx], b[i]));  // two roundings, as the contract's expression reads
}

bool fits31(uint64_t v) { return v > 0 && v <= 0x7FFFFFFFull; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

}  // namespace tsr

using namespace tsr;

extern "C" {

int tsr_moe_gate(const float* vals, const float* x, const float* w, float* wts, float* sig, uint64_t top_k,
                 uint64_t hidden, void* stream) {
  if (!vals || !x || !w || !wts || !sig || !fits31(top_k) || !fits31(hidden)) return kInvalidArgument;
  moe_gate_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(vals, x, w, wts, sig, static_cast<int>(top_k),
                                                                     static_cast<int>(hidden));
  return check_launch();
}

int tsr_moe_scale_add(const float* a, const float* b, const float* f, float* o, uint64_t n, uint64_t idx, void* stream) {
  if (!a || !b || !f || !o || n == 0) return kInvalidArgument;
  moe_scale_add_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b, f, o, n,
                                                                                                                   idx);
  return check_launch();
}

int tsr_moe_experts_gate_up_q4k(const float* x, const void* gate, const void* up, const uint32_t* ids, float* phi,
                                uint64_t hidden, uint64_t inter, uint64_t top_k, uint64_t gate_stride, uint64_t up_stride,
                                uint64_t experts, void* stream) {
  if (!x || !gate || !up || !ids || !phi || !fits31(hidden) || !fits31(inter) || !fits31(top_k) || !fits31(experts) ||
      hidden % 256 != 0 || !fits31(inter * top_k) || hidden * 4 > 200 * 1024)
    return kInvalidArgument;
  if (!aligned16(x) || !aligned16(gate) || !aligned16(up) || gate_stride % 16 != 0 || up_stride % 16 != 0)
    return kInvalidArgument;
  const size_t smem = hidden * 4;
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&moe_gate_up_q4k_kernel), 227 * 1024)) return rc;
  const unsigned blocks = static_cast<unsigned>((inter * top_k + kMoeWarps - 1) / kMoeWarps);
  moe_gate_up_q4k_kernel<<<blocks, kMoeWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<const uint8_t*>(gate), static_cast<const uint8_t*>(up), ids, phi, static_cast<int>(hidden),
      static_cast<int>(inter), static_cast<int>(top_k), gate_stride, up_stride, static_cast<int>(experts));
  return check_launch();
}

int tsr_moe_experts_down(int fmt, const float* phi, const void* down, const uint32_t* ids, const float* wts, float* out,
                         uint64_t hidden, uint64_t inter, uint64_t top_k, uint64_t down_stride, uint64_t accumulate,
                         uint64_t experts, void* stream) {
  if ((fmt != 0 && fmt != 1) || !phi || !down || !ids || !wts || !out || !fits31(hidden) || !fits31(inter) ||
      !fits31(top_k) || !fits31(experts) || inter % 256 != 0 || top_k * inter * 4 > 200 * 1024)
    return kInvalidArgument;
  if (!aligned16(phi) || (fmt == 0 && (!aligned16(down) || down_stride % 16 != 0)) ||
      (fmt == 1 && ((reinterpret_cast<uintptr_t>(down) & 1u) || down_stride % 2 != 0)))
    return kInvalidArgument;
  const size_t smem = top_k * inter * 4;
  const unsigned blocks = static_cast<unsigned>((hidden + kMoeWarps - 1) / kMoeWarps);
  auto st = static_cast<cudaStream_t>(stream);
  if (fmt == 0) {
    if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&moe_down_kernel<false>), 227 * 1024)) return rc;
    moe_down_kernel<false><<<blocks, kMoeWarps * 32, smem, st>>>(phi, static_cast<const uint8_t*>(down), ids, wts, out,
                                                                  static_cast<int>(hidden), static_cast<int>(inter),
                                                                  static_cast<int>(top_k), down_stride,
                                                                  accumulate != 0 ? 1 : 0, static_cast<int>(experts));
  } else {
    if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&moe_down_kernel<true>), 227 * 1024)) return rc;
    moe_down_kernel<true><<<blocks, kMoeWarps * 32, smem, st>>>(phi, static_cast<const uint8_t*>(down), ids, wts, out,
                                                                 static_cast<int>(hidden), static_cast<int>(inter),
                                                                 static_cast<int>(top_k), down_stride,
                                                                 accumulate != 0 ? 1 : 0, static_cast<int>(experts));
  }
  return check_launch();
}

}  // extern "C"
