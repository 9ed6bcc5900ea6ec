// Elementwise and row-wise steps of the reference's forward that sit between the
// projections (src/models/qwen3_5/trunk.cpp:486-501 loads them by these ids):
// sigmoid_gate, l2norm, rmsnorm_gated, ssm_gate, qgate_split, repeat_heads.
// Contracts: include/tessera/backend.hpp:217-254,386-390 of the reference; arithmetic:
// src/core/numerics/norm.cpp:96-262 and attention.cpp:290-334 (the *Ref functions).
// All of them move a few KB to a few hundred KB per token: one pass, coalesced, fp32.
#include <cuda_fp16.h>

#include "codec.cuh"
#include "launch.h"
#include "tessera_b200.h"

namespace tsr {
namespace {

// O = A * sigmoid(G) (SigmoidGateRef: a / (1 + exp(-g)))
__global__ void sigmoid_gate_kernel(const float* __restrict__ a, const float* __restrict__ g, float* __restrict__ o,
                                    size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) o[i] = a[i] / (1.0f + expf(-g[i]));
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// Y = scale * X / sqrt(sum(X^2) + eps), one CTA per row (L2NormRef; the squares are added as a tree)
__global__ void __launch_bounds__(256)
l2norm_kernel(const float* __restrict__ x, float* __restrict__ y, int cols, float eps, float scale) {
  __shared__ float red[32];
  const float* row = x + static_cast<size_t>(blockIdx.x) * cols;
  float s = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s = fmaf(row[c], row[c], s);
  const float gain = scale / sqrtf(block_sum(s, red) + eps);
  float* out = y + static_cast<size_t>(blockIdx.x) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) out[c] = row[c] * gain;
}

// Y[ybase + r*cols + c] = X[r*cols + c] / sqrt(mean(X_r^2) + eps) * W[c] * silu(G[gbase + r*cols + c])
// (RmsNormGatedRef; the bases address one token's slice of a batched buffer)
__global__ void __launch_bounds__(256)
rmsnorm_gated_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ gate,
                     float* __restrict__ y, int cols, float eps, size_t gbase, size_t ybase) {
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * cols;
  const float* row = x + base;
  float s = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s = fmaf(row[c], row[c], s);
  const float gain = 1.0f / sqrtf(block_sum(s, red) / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float g = gate[gbase + base + c];
    const float silu = g / (1.0f + expf(-g));
    y[ybase + base + c] = row[c] * gain * w[c] * silu;
  }
}

// alpha = exp(a_log[h] * softplus(alpha_raw + dt[h])), beta = sigmoid(beta_raw) (SsmGateRef)
__global__ void ssm_gate_kernel(const float* __restrict__ a_log, const float* __restrict__ dt,
                                const float* __restrict__ alpha_raw, const float* __restrict__ beta_raw,
                                float* __restrict__ alpha, float* __restrict__ beta, size_t heads, size_t total) {
  const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const size_t h = t % heads;
  const float raw = alpha_raw[t] + dt[h];
  const float softplus = raw > 20.0f ? raw : log1pf(expf(raw));
  alpha[t] = expf(a_log[h] * softplus);
  beta[t] = 1.0f / (1.0f + expf(-beta_raw[t]));
}

// fused[(r*heads + h)*2*d + e] -> q[(r*heads + h)*d + e], fused[... + d + e] -> gate[...] (QGateSplitRef)
__global__ void qgate_split_kernel(const float* __restrict__ fused, float* __restrict__ q, float* __restrict__ gate,
                                   size_t head_dim, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t rh = i / head_dim, e = i - rh * head_dim;
  const float* src = fused + rh * 2 * head_dim;
  q[i] = src[e];
  gate[i] = src[head_dim + e];
}

// out[r][h][e] = in[r][h % (num_v_heads / factor)][e] (RepeatHeadsRef, row by row)
__global__ void repeat_heads_kernel(const float* __restrict__ in, float* __restrict__ out, size_t num_v_heads,
                                    size_t head_k_dim, size_t num_k_heads, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t e = i % head_k_dim, rh = i / head_k_dim;
  const size_t h = rh % num_v_heads, r = rh / num_v_heads;
  out[i] = in[(r * num_k_heads + h % num_k_heads) * head_k_dim + e];
}

// Out[row] = table[ids[row]] as fp32, a zero row for an id outside the table
// (include/tessera/backend.hpp:261-265).  KIND 0: fp32 table, 1: bf16, 2: Q4_K rows of cols/256
// blocks, decoded with the reference's rounding sequence (src/core/numerics/quant.cpp:656-675).
template <int KIND>
__global__ void embedding_kernel(const uint32_t* __restrict__ ids, const uint8_t* __restrict__ table,
                                 float* __restrict__ out, size_t cols, size_t vocab, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / cols, t = i - r * cols;
  const size_t id = ids[r];
  float v = 0.0f;
  if (id < vocab) {
    if (KIND == 0) {
      v = reinterpret_cast<const float*>(table)[id * cols + t];
    } else if (KIND == 1) {
      v = __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(table)[id * cols + t]) << 16);
    } else {
      const uint8_t* blk = table + (id * (cols / 256) + t / 256) * kQ4KBlockBytes;
      const int e = static_cast<int>(t % 256), g = e / 64, hi = (e % 64) / 32, l = e % 32;
      const float d = fp16_bits_to_float(blk[0] | (blk[1] << 8));
      const float dmin = fp16_bits_to_float(blk[2] | (blk[3] << 8));
      uint32_t s[3];
      for (int w = 0; w < 3; ++w)
        s[w] = blk[4 + 4 * w] | (blk[5 + 4 * w] << 8) | (blk[6 + 4 * w] << 16) | (static_cast<uint32_t>(blk[7 + 4 * w]) << 24);
      uint32_t sc, mn;
      q4k_scale_min(s, 2 * g + hi, sc, mn);
      const uint32_t byte = blk[16 + 32 * g + l];
      const float q = static_cast<float>(hi ? (byte >> 4) : (byte & 15u));
      v = __fsub_rn(__fmul_rn(__fmul_rn(d, static_cast<float>(sc)), q), __fmul_rn(dmin, static_cast<float>(mn)));
    }
  }
  out[i] = v;
}

// mrope: rows x heads x head_dim fp32 rotated in place, NeoX pairing (j, j + rope_dim/2); pair j turns
// by pos[section of j] * theta^(-2j / rope_dim) (MropeRef, src/core/numerics/attention.cpp: the angle,
// its cosine and sine in double precision, then fp32 products).
__global__ void mrope_kernel(float* __restrict__ io, const unsigned long long* __restrict__ pos, size_t heads,
                             size_t head_dim, size_t rope_dim, double theta, size_t sec_t, size_t sec_h, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t pairs = rope_dim / 2;
  const size_t j = i % pairs, rh = i / pairs, r = rh / heads;
  const unsigned long long section_pos = j < sec_t ? pos[r * 3] : j < sec_t + sec_h ? pos[r * 3 + 1] : pos[r * 3 + 2];
  const double angle = static_cast<double>(section_pos) *
                       pow(theta, -2.0 * static_cast<double>(j) / static_cast<double>(rope_dim));
  const float c = static_cast<float>(cos(angle)), sn = static_cast<float>(sin(angle));
  float* base = io + rh * head_dim;
  const float x1 = base[j], x2 = base[j + pairs];
  base[j] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
  base[j + pairs] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, c));
}

// rope: the same rotation with one position per row, pos_base + r (RopeRef, src/core/numerics/attention.cpp:11-43)
__global__ void rope_kernel(float* __restrict__ io, size_t heads, size_t head_dim, size_t rope_dim, unsigned long long pos_base,
                            double theta, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t pairs = rope_dim / 2;
  const size_t j = i % pairs, rh = i / pairs, r = rh / heads;
  const double angle = static_cast<double>(pos_base + r) * pow(theta, -2.0 * static_cast<double>(j) / static_cast<double>(rope_dim));
  const float c = static_cast<float>(cos(angle)), sn = static_cast<float>(sin(angle));
  float* base = io + rh * head_dim;
  const float x1 = base[j], x2 = base[j + pairs];
  base[j] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
  base[j + pairs] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, c));
}

// quantize_q8 / quantize_q4: one CTA per row; scale = amax / LIMIT (1 for a zero row), codes
// round-half-away(x / scale) clamped to +-LIMIT; int8 bytes, or nibbles with element 2i in the low half
// (QuantizeQ8Ref, QuantizeQ4Ref, src/core/numerics/quant.cpp:123-181).  Bit-equal: max is exact in any order.
template <int LIMIT>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const float* __restrict__ in, unsigned char* __restrict__ out, float* __restrict__ scale, int cols) {
  __shared__ float red[8];
  const float* row = in + static_cast<size_t>(blockIdx.x) * cols;
  float amax = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(row[c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float s = amax > 0.0f ? __fdiv_rn(amax, static_cast<float>(LIMIT)) : 1.0f;
  if (threadIdx.x == 0) scale[blockIdx.x] = s;
  auto code = [&](int c) {
    const float q = fminf(fmaxf(roundf(__fdiv_rn(row[c], s)), -static_cast<float>(LIMIT)), static_cast<float>(LIMIT));
    return static_cast<unsigned>(static_cast<int>(q));
  };
  if (LIMIT == 127) {  // four bytes per thread and trip
    uint32_t* o = reinterpret_cast<uint32_t*>(out + static_cast<size_t>(blockIdx.x) * cols);
    for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4)
      o[c / 4] = (code(c) & 0xFFu) | ((code(c + 1) & 0xFFu) << 8) | ((code(c + 2) & 0xFFu) << 16) | ((code(c + 3) & 0xFFu) << 24);
  } else {  // eight nibbles
    uint32_t* o = reinterpret_cast<uint32_t*>(out + static_cast<size_t>(blockIdx.x) * cols / 2);
    for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) word |= (code(c + e) & 0xFu) << (4 * e);
      o[c / 8] = word;
    }
  }
}

// fp32 -> binary16, round to nearest even, two per 32-bit word (backend.hpp:334-336)
__global__ void cast_f32_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2half_rn(in[i]);
}

// delta_step_heads: the gated delta rule, `rows` steps in turn on the recurrent state of every
// value head (DeltaStepHeadsRef, attention.cpp; indexing of the device contract,
// src/backends/rocm/rocm_kernels_basic.cpp: the state is read at sbase, row t's updated state
// goes to sbase + (t+1)*sstride, or back in place after the last row when sstride is 0; alpha
// and beta are read at abase + t*heads + h).
//   r = S^T k;  S' = alpha (S - beta k r^T) + beta k v^T;  o = S'^T q     per head
// A CTA owns 32 state columns of one head: warp w holds rows j = w*dk/4 .. of those columns in
// registers (lane = column, so every state access is a 128-byte row segment), the four warps'
// partial sums meet in shared memory.  HBM-bound: the state (heads x dk x dv fp32: 3 MB per layer
// at 48 x 128 x 128) is read once and written once per call.
constexpr int kDeltaCols = 32, kDeltaWarps = 4, kDeltaMaxPer = 64;  // dk <= 256 (eight warps measured slower: 6.4 against 5.0 us)
__global__ void __launch_bounds__(kDeltaCols * kDeltaWarps)
delta_step_heads_kernel(float* __restrict__ s, const float* __restrict__ k, const float* __restrict__ v,
                        const float* __restrict__ q, float* __restrict__ o, const float* __restrict__ alpha,
                        const float* __restrict__ beta, int heads, int dk, int dv, int rows, size_t sbase,
                        size_t sstride, size_t abase) {
  __shared__ float part[kDeltaWarps][kDeltaCols];
  __shared__ float kq[2][256];
  const int slabs = (dv + kDeltaCols - 1) / kDeltaCols;
  const int h = blockIdx.x / slabs, d = (blockIdx.x % slabs) * kDeltaCols + (threadIdx.x & 31);
  const int w = threadIdx.x >> 5;
  const int per = (dk + kDeltaWarps - 1) / kDeltaWarps, j0 = w * per;
  const int jn = max(0, min(dk, j0 + per) - j0);
  const bool col = d < dv;
  float st[kDeltaMaxPer];
  const size_t head_state = static_cast<size_t>(h) * dk * dv;
#pragma unroll
  for (int jj = 0; jj < kDeltaMaxPer; ++jj)
    st[jj] = (jj < jn && col) ? s[sbase + head_state + static_cast<size_t>(j0 + jj) * dv + d] : 0.0f;
  for (int t = 0; t < rows; ++t) {
    const size_t ko = (static_cast<size_t>(t) * heads + h) * dk, vo = (static_cast<size_t>(t) * heads + h) * dv;
    __syncthreads();  // the previous row's readers of kq and part are done
    for (int j = threadIdx.x; j < dk; j += blockDim.x) {
      kq[0][j] = k[ko + j];
      kq[1][j] = q[ko + j];
    }
    __syncthreads();
    const float a = alpha[abase + static_cast<size_t>(t) * heads + h], b = beta[abase + static_cast<size_t>(t) * heads + h];
    const float vb = col ? v[vo + d] : 0.0f;
    float r = 0.0f;
#pragma unroll
    for (int jj = 0; jj < kDeltaMaxPer; ++jj)
      if (jj < jn) r = fmaf(st[jj], kq[0][j0 + jj], r);
    part[w][threadIdx.x & 31] = r;
    __syncthreads();
    float read = 0.0f;
#pragma unroll
    for (int x = 0; x < kDeltaWarps; ++x) read += part[x][threadIdx.x & 31];
    float out = 0.0f;
#pragma unroll
    for (int jj = 0; jj < kDeltaMaxPer; ++jj)
      if (jj < jn) {
        const float kk = kq[0][j0 + jj];
        st[jj] = a * (st[jj] - b * kk * read) + b * vb * kk;
        out = fmaf(st[jj], kq[1][j0 + jj], out);
      }
    __syncthreads();  // everybody has read `part`
    part[w][threadIdx.x & 31] = out;
    __syncthreads();
    if (w == 0 && col) {
      float sum = 0.0f;
#pragma unroll
      for (int x = 0; x < kDeltaWarps; ++x) sum += part[x][threadIdx.x & 31];
      o[vo + d] = sum;
    }
    if (sstride != 0 && col) {
#pragma unroll
      for (int jj = 0; jj < kDeltaMaxPer; ++jj)
        if (jj < jn) s[sbase + (static_cast<size_t>(t) + 1) * sstride + head_state + static_cast<size_t>(j0 + jj) * dv + d] = st[jj];
    }
  }
  if (sstride == 0 && col) {
#pragma unroll
    for (int jj = 0; jj < kDeltaMaxPer; ++jj)
      if (jj < jn) s[sbase + head_state + static_cast<size_t>(j0 + jj) * dv + d] = st[jj];
  }
}

// conv1d_state: current-step causal depthwise convolution with the history kept on the device, SiLU and
// the q / k / v split; `rows` steps advance the history in turn.  One thread per channel; W in checkpoint
// tap order (tap 0 oldest), history newest first, (width - 1) samples per channel; with hist_stride != 0
// row t's history also goes to slot t + 1 of hist_hist (device contract:
// src/backends/rocm/rocm_kernels_basic.cpp:2193-2245 of the reference; the convolution itself is
// Conv1dStepRef, src/core/numerics/conv.cpp).
__global__ void conv1d_state_kernel(const float* __restrict__ qkv, const float* __restrict__ w, float* __restrict__ hist,
                                    float* __restrict__ q, float* __restrict__ k, float* __restrict__ v,
                                    float* __restrict__ hist_hist, size_t conv_dim, size_t width, size_t key_dim,
                                    size_t qkv_offset, size_t rows, size_t hist_stride) {
  const size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= conv_dim) return;
  const size_t stride = width - 1, hbase = c * stride, value_dim = conv_dim - 2 * key_dim;
  for (size_t t = 0; t < rows; ++t) {
    const float current = qkv[qkv_offset + t * conv_dim + c];
    float acc = __fmul_rn(w[c * width + (width - 1)], current);
    for (size_t i = 1; i < width; ++i) acc = fmaf(w[c * width + (width - 1 - i)], hist[hbase + (i - 1)], acc);
    const float out = acc / (1.0f + expf(-acc));
    if (c < key_dim) q[t * key_dim + c] = out;
    else if (c < 2 * key_dim) k[t * key_dim + (c - key_dim)] = out;
    else v[t * value_dim + (c - 2 * key_dim)] = out;
    if (width > 1) {
      for (size_t i = stride; i > 1; --i) hist[hbase + (i - 1)] = hist[hbase + (i - 2)];
      hist[hbase] = current;
    }
    if (hist_stride != 0)
      for (size_t i = 0; i < stride; ++i) hist_hist[(t + 1) * hist_stride + hbase + i] = hist[hbase + i];
  }
}

// The steps between a linear-attention layer's input projections and its state step in one launch: CTA b takes
// channels [b cols, (b + 1) cols) of the convolution (cols = the heads' width = blockDim): the first k_heads CTAs
// are the q heads, the next k_heads the k heads (convolution, SiLU, l2norm of the head, the head repeated into the
// expanded layout), the rest value channels (convolution and SiLU); one more CTA evaluates ssm_gate.  Same
// arithmetic and the same order of additions as conv1d_state_kernel, l2norm_kernel, repeat_heads_kernel and
// ssm_gate_kernel.
__global__ void __launch_bounds__(1024) linear_mixer_inputs_kernel(const LinearMixerInputs p) {
  __shared__ float red[32];
  const int b = blockIdx.x, tid = threadIdx.x;
  if (b == static_cast<int>(gridDim.x) - 1) {
    for (int h = tid; h < p.gate_heads; h += blockDim.x) {
      const float raw = p.alpha_raw[h] + p.dt[h];
      const float softplus = raw > 20.0f ? raw : log1pf(expf(raw));
      p.alpha[h] = expf(p.a_log[h] * softplus);
      p.beta[h] = 1.0f / (1.0f + expf(-p.beta_raw[h]));
    }
    return;
  }
  const size_t c = static_cast<size_t>(b) * p.cols + tid;
  const size_t stride = p.width - 1, hbase = c * stride;
  const float current = p.qkv[p.qkv_offset + c];
  float acc = __fmul_rn(p.conv_w[c * p.width + (p.width - 1)], current);
  for (int i = 1; i < p.width; ++i) acc = fmaf(p.conv_w[c * p.width + (p.width - 1 - i)], p.hist[hbase + (i - 1)], acc);
  const float out = acc / (1.0f + expf(-acc));
  if (p.width > 1) {
    for (size_t i = stride; i > 1; --i) p.hist[hbase + (i - 1)] = p.hist[hbase + (i - 2)];
    p.hist[hbase] = current;
  }
  if (b >= 2 * p.k_heads) {
    p.v[c - 2 * static_cast<size_t>(p.key_dim)] = out;
    return;
  }
  const bool is_k = b >= p.k_heads;
  const int head = is_k ? b - p.k_heads : b;
  const float sum = block_sum(fmaf(out, out, 0.0f), red);
  const float gain = (is_k ? p.scale_k : p.scale_q) / sqrtf(sum + (is_k ? p.eps_k : p.eps_q));
  const float y = out * gain;
  (is_k ? p.k : p.q)[static_cast<size_t>(head) * p.cols + tid] = y;
  float* expanded = is_k ? p.k_exp : p.q_exp;
  for (int j = 0; j < p.factor; ++j) expanded[(static_cast<size_t>(j) * p.k_heads + head) * p.cols + tid] = y;
}

// The steps between a full-attention layer's q / k / v projections and its attention in one launch: CTA r is one
// head of q (r < heads) or of k: rmsnorm of the head with the per-head weight, mrope of the normalised head, both
// in place, the k heads also written to their cache row; one more CTA copies the token's v row to the cache.
// Same arithmetic and order of additions as rmsnorm_kernel and mrope_kernel.
__global__ void __launch_bounds__(1024) head_norm_rope_kernel(const HeadNormRope p) {
  __shared__ float red[32];
  __shared__ float normed[1024];
  const int r = blockIdx.x, tid = threadIdx.x;
  if (r == p.heads + p.kv_heads) {
    for (int t = tid; t < p.kv_heads * p.head_dim; t += blockDim.x) p.v_row[t] = p.v_src[t];
    return;
  }
  const bool is_k = r >= p.heads;
  float* row = is_k ? p.k + static_cast<size_t>(r - p.heads) * p.head_dim : p.q + static_cast<size_t>(r) * p.head_dim;
  float* cache = is_k && p.k_row != nullptr ? p.k_row + static_cast<size_t>(r - p.heads) * p.head_dim : nullptr;
  const float x = row[tid];
  const float sum = block_sum(fmaf(x, x, 0.0f), red);
  const float gain = 1.0f / sqrtf(sum / static_cast<float>(p.head_dim) + (is_k ? p.eps_k : p.eps_q));
  const float y = x * gain * (is_k ? p.k_w : p.q_w)[tid];
  normed[tid] = y;
  __syncthreads();
  const int pairs = p.rope_dim / 2;
  if (tid < pairs) {
    const int j = tid;
    const unsigned long long section_pos = j < p.sec_t ? p.pos[0] : j < p.sec_t + p.sec_h ? p.pos[1] : p.pos[2];
    const double angle = static_cast<double>(section_pos) *
                         pow(static_cast<double>(p.theta), -2.0 * static_cast<double>(j) / static_cast<double>(p.rope_dim));
    const float c = static_cast<float>(cos(angle)), sn = static_cast<float>(sin(angle));
    const float x1 = normed[j], x2 = normed[j + pairs];
    const float o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)), o2 = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, c));
    row[j] = o1, row[j + pairs] = o2;
    if (cache != nullptr) cache[j] = o1, cache[j + pairs] = o2;
  } else if (tid >= p.rope_dim) {
    row[tid] = y;
    if (cache != nullptr) cache[tid] = y;
  }
}

// top_k_rows: the top_k (<= 32) largest of `vocab` fp32 logits of every row, descending, with their
// indices; output row r reads input row row_base + r (src/backends/rocm/rocm_kernels.hpp:558-566).  One
// CTA per row; top_k rounds of a block-wide arg-max over the values not taken yet; among equal values the
// lowest index wins.
__global__ void __launch_bounds__(256)
top_k_rows_kernel(const float* __restrict__ logits, uint32_t* __restrict__ ids, float* __restrict__ vals, size_t vocab,
                  int top_k, size_t row_base) {
  __shared__ float bv[8];
  __shared__ uint32_t bi[8];
  __shared__ uint32_t taken[32];
  const float* row = logits + (row_base + blockIdx.x) * vocab;
  for (int p = 0; p < top_k; ++p) {
    float best = -INFINITY;
    uint32_t arg = 0xFFFFFFFFu;
    for (size_t c = threadIdx.x; c < vocab; c += blockDim.x) {
      const float x = row[c];
      bool used = false;
      for (int t = 0; t < p; ++t) used = used || taken[t] == static_cast<uint32_t>(c);
      if (!used && (x > best || (x == best && static_cast<uint32_t>(c) < arg) || arg == 0xFFFFFFFFu)) {
        best = x;
        arg = static_cast<uint32_t>(c);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, arg, o);
      if (oi != 0xFFFFFFFFu && (arg == 0xFFFFFFFFu || ov > best || (ov == best && oi < arg))) {
        best = ov;
        arg = oi;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      bv[threadIdx.x >> 5] = best;
      bi[threadIdx.x >> 5] = arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int x = 1; x < 8; ++x)
        if (bi[x] != 0xFFFFFFFFu && (bi[0] == 0xFFFFFFFFu || bv[x] > bv[0] || (bv[x] == bv[0] && bi[x] < bi[0]))) {
          bv[0] = bv[x];
          bi[0] = bi[x];
        }
      taken[p] = bi[0];
      vals[blockIdx.x * top_k + p] = bi[0] == 0xFFFFFFFFu ? -INFINITY : bv[0];
      ids[blockIdx.x * top_k + p] = bi[0] == 0xFFFFFFFFu ? 0u : bi[0];
    }
    __syncthreads();
  }
}

unsigned blocks_of(size_t n) { return static_cast<unsigned>((n + 255) / 256); }
bool fits31(uint64_t v) { return v > 0 && v <= 0x7FFFFFFFull; }

}  // namespace

int launch_linear_mixer_inputs(const LinearMixerInputs& p, cudaStream_t st) {
  if (p.cols <= 0 || p.cols > 1024 || p.cols % 32 != 0 || p.conv_dim % p.cols != 0) return kUnsupportedFeature;
  linear_mixer_inputs_kernel<<<static_cast<unsigned>(p.conv_dim / p.cols + 1), static_cast<unsigned>(p.cols), 0, st>>>(p);
  return check_launch();
}

int launch_head_norm_rope(const HeadNormRope& p, cudaStream_t st) {
  if (p.head_dim <= 0 || p.head_dim > 1024 || p.head_dim % 32 != 0) return kUnsupportedFeature;
  const unsigned grid = static_cast<unsigned>(p.heads + p.kv_heads + (p.v_row != nullptr ? 1 : 0));
  head_norm_rope_kernel<<<grid, static_cast<unsigned>(p.head_dim), 0, st>>>(p);
  return check_launch();
}
}  // namespace tsr

using namespace tsr;

extern "C" {

int tsr_sigmoid_gate(const float* a, const float* g, float* o, uint64_t n, void* stream) {
  if (!a || !g || !o || n == 0) return kInvalidArgument;
  sigmoid_gate_kernel<<<blocks_of(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, g, o, n);
  return check_launch();
}

int tsr_l2norm(const float* x, float* y, uint64_t rows, uint64_t cols, float eps, float scale, void* stream) {
  if (!x || !y || !fits31(rows) || !fits31(cols) || !(eps >= 0.0f)) return kInvalidArgument;
  l2norm_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, static_cast<int>(cols),
                                                                                            eps, scale);
  return check_launch();
}

int tsr_rmsnorm_gated(const float* x, const float* w, const float* gate, float* y, uint64_t rows, uint64_t cols,
                      float eps, uint64_t gbase, uint64_t ybase, void* stream) {
  if (!x || !w || !gate || !y || !fits31(rows) || !fits31(cols) || !(eps >= 0.0f)) return kInvalidArgument;
  rmsnorm_gated_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, w, gate, y, static_cast<int>(cols), eps, gbase, ybase);
  return check_launch();
}

int tsr_ssm_gate(const float* a_log, const float* dt, const float* alpha_raw, const float* beta_raw, float* alpha,
                 float* beta, uint64_t heads, uint64_t rows, void* stream) {
  if (!a_log || !dt || !alpha_raw || !beta_raw || !alpha || !beta || !fits31(heads) || !fits31(rows)) return kInvalidArgument;
  const size_t total = heads * rows;
  ssm_gate_kernel<<<blocks_of(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(a_log, dt, alpha_raw, beta_raw, alpha,
                                                                                    beta, heads, total);
  return check_launch();
}

int tsr_qgate_split(const float* fused, float* q, float* gate, uint64_t heads, uint64_t head_dim, uint64_t rows,
                    void* stream) {
  if (!fused || !q || !gate || !fits31(heads) || !fits31(head_dim) || !fits31(rows)) return kInvalidArgument;
  const size_t total = rows * heads * head_dim;
  qgate_split_kernel<<<blocks_of(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(fused, q, gate, head_dim, total);
  return check_launch();
}

int tsr_embedding(int kind, const uint32_t* ids, const void* table, float* out, uint64_t rows, uint64_t cols,
                  uint64_t vocab, void* stream) {
  if (!ids || !table || !out || !fits31(rows) || !fits31(cols) || !fits31(vocab) || kind < 0 || kind > 2 ||
      (kind == 2 && cols % 256 != 0))
    return kInvalidArgument;
  const size_t total = rows * cols;
  auto st = static_cast<cudaStream_t>(stream);
  auto* t = static_cast<const uint8_t*>(table);
  if (kind == 0) embedding_kernel<0><<<blocks_of(total), 256, 0, st>>>(ids, t, out, cols, vocab, total);
  else if (kind == 1) embedding_kernel<1><<<blocks_of(total), 256, 0, st>>>(ids, t, out, cols, vocab, total);
  else embedding_kernel<2><<<blocks_of(total), 256, 0, st>>>(ids, t, out, cols, vocab, total);
  return check_launch();
}

int tsr_mrope(float* io, const uint64_t* pos, uint64_t rows, uint64_t heads, uint64_t head_dim, uint64_t rope_dim,
              float theta, uint64_t sec_t, uint64_t sec_h, uint64_t sec_w, void* stream) {
  if (!io || !pos || !fits31(rows) || !fits31(heads) || !fits31(head_dim) || rope_dim == 0 || rope_dim > head_dim ||
      head_dim % 2 != 0 || rope_dim % 2 != 0 || sec_t + sec_h + sec_w > rope_dim / 2 || !(theta > 0.0f))
    return kInvalidArgument;
  const size_t total = rows * heads * (rope_dim / 2);
  mrope_kernel<<<blocks_of(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      io, reinterpret_cast<const unsigned long long*>(pos), heads, head_dim, rope_dim, static_cast<double>(theta), sec_t,
      sec_h, total);
  return check_launch();
}

int tsr_rope(float* io, uint64_t rows, uint64_t heads, uint64_t head_dim, uint64_t rope_dim, uint64_t pos_base, float theta,
             void* stream) {
  if (!io || !fits31(rows) || !fits31(heads) || !fits31(head_dim) || rope_dim == 0 || rope_dim > head_dim || rope_dim % 2 != 0 ||
      !(theta > 0.0f))
    return kInvalidArgument;
  const size_t total = rows * heads * (rope_dim / 2);
  rope_kernel<<<blocks_of(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(io, heads, head_dim, rope_dim, pos_base,
                                                                             static_cast<double>(theta), total);
  return check_launch();
}

int tsr_quantize_rows(int kind, const float* in, void* out, float* scale, uint64_t rows, uint64_t cols, void* stream) {
  if (!in || !out || !scale || !fits31(rows) || !fits31(cols) || (kind != 0 && kind != 1) || cols % (kind == 0 ? 4 : 8) != 0)
    return kInvalidArgument;
  auto st = static_cast<cudaStream_t>(stream);
  if (kind == 0)
    quantize_rows_kernel<127><<<static_cast<unsigned>(rows), 256, 0, st>>>(in, static_cast<unsigned char*>(out), scale,
                                                                          static_cast<int>(cols));
  else
    quantize_rows_kernel<7><<<static_cast<unsigned>(rows), 256, 0, st>>>(in, static_cast<unsigned char*>(out), scale,
                                                                        static_cast<int>(cols));
  return check_launch();
}

int tsr_cast_f32_f16(const float* in, void* out, uint64_t n, void* stream) {
  if (!in || !out || n == 0 || n % 2 != 0) return kInvalidArgument;
  cast_f32_f16_kernel<<<blocks_of(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, static_cast<__half*>(out), n);
  return check_launch();
}

int tsr_delta_step_heads(float* s, const float* k, const float* v, const float* q, float* o, const float* alpha,
                         const float* beta, uint64_t heads, uint64_t dk, uint64_t dv, uint64_t rows, uint64_t sbase,
                         uint64_t sstride, uint64_t abase, void* stream) {
  if (!s || !k || !v || !q || !o || !alpha || !beta || !fits31(heads) || !fits31(dk) || !fits31(dv) || !fits31(rows) ||
      dk > 256)
    return kInvalidArgument;
  const unsigned slabs = static_cast<unsigned>((dv + kDeltaCols - 1) / kDeltaCols);
  delta_step_heads_kernel<<<static_cast<unsigned>(heads) * slabs, kDeltaCols * kDeltaWarps, 0,
                            static_cast<cudaStream_t>(stream)>>>(s, k, v, q, o, alpha, beta, static_cast<int>(heads),
                                                                 static_cast<int>(dk), static_cast<int>(dv),
                                                                 static_cast<int>(rows), sbase, sstride, abase);
  return check_launch();
}

int tsr_conv1d_state(const float* qkv, const float* w, float* hist, float* q, float* k, float* v, float* hist_hist,
                     uint64_t conv_dim, uint64_t width, uint64_t key_dim, uint64_t qkv_offset, uint64_t rows,
                     uint64_t hist_stride, void* stream) {
  if (!qkv || !w || !hist || !q || !k || !v || !fits31(conv_dim) || !fits31(width) || !fits31(rows) || 2 * key_dim > conv_dim ||
      (hist_stride != 0 && !hist_hist))
    return kInvalidArgument;
  conv1d_state_kernel<<<blocks_of(conv_dim), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      qkv, w, hist, q, k, v, hist_hist, conv_dim, width, key_dim, qkv_offset, rows, hist_stride);
  return check_launch();
}

int tsr_top_k_rows(const float* logits, uint32_t* ids, float* vals, uint64_t rows, uint64_t vocab, uint64_t top_k,
                   uint64_t row_base, void* stream) {
  if (!logits || !ids || !vals || !fits31(rows) || !fits31(vocab) || top_k == 0 || top_k > 32) return kInvalidArgument;
  top_k_rows_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, ids, vals, vocab, static_cast<int>(top_k), row_base);
  return check_launch();
}

int tsr_repeat_heads(const float* in, float* out, uint64_t num_v_heads, uint64_t head_k_dim, uint64_t factor,
                     uint64_t rows, void* stream) {
  if (!in || !out || !fits31(num_v_heads) || !fits31(head_k_dim) || !fits31(factor) || !fits31(rows) ||
      num_v_heads % factor != 0)
    return kInvalidArgument;
  const size_t total = rows * num_v_heads * head_k_dim;
  repeat_heads_kernel<<<blocks_of(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, num_v_heads, head_k_dim,
                                                                                        num_v_heads / factor, total);
  return check_launch();
}

}  // extern "C"
