// Causal grouped-query attention of a few query rows over the key/value cache
// (the decode and verify steps): ids "attention" (fp32 or fp16 cache) and
// "attention_q8" / "attention_q4" / "attention_fp8" (int8 / 4-bit / OCP FP8 E4M3
// cache with one fp32 scale per key position).  Contracts: include/tessera/backend.hpp:167-179,283-309 of the
// reference; arithmetic: AttentionRef, AttentionRefF16, AttentionQ8Ref, AttentionQ4Ref, AttentionFp8Ref
// (src/core/numerics/attention.cpp): scores q.k / sqrt(head_dim) over keys
// start..last of the causal window, softmax, weighted sum of the values; query
// head h reads kv head h / (heads / kv_heads).
//
// HBM-bound over the cache (context 4096, 4 kv heads of 256: 32 MB in fp32, 8 MB in
// FP8 per layer and token), with 4 head_dim G multiply-adds per key and kv head on
// the fp32 pipe beside it.  The key range is cut into chunks (flash decoding): a
// CTA takes one kv head, one query row and one chunk and serves all query heads
// of the group from one pass over its keys; a second small kernel merges the
// chunks.  The halves are also ids of their own ("attention_split",
// "attention_split_gqa", "attention_q8_split" ..., "attention_combine") with the
// reference's partial layout, because the reference's single-token path calls
// them with its own chunk count and buffers (src/core/decode_internal.hpp:299-374).
#include <cuda_fp16.h>

#include "codec.cuh"
#include "launch.h"
#include "tessera_b200.h"

namespace tsr {
namespace {

constexpr int kAttnWarps = 8, kAttnMaxGroup = 8;  // heads / kv_heads <= 8
constexpr int kAttnMaxSplits = 64, kAttnMinKeys = 64;  // chunks the whole-attention entry cuts the key range into
constexpr float kNullMax = -1e30f;  // running max before the first key, as the reference's kernels have it

enum : int { kKvF32 = 0, kKvF16 = 1, kKvFp8 = 2, kKvInt8 = 3, kKvInt4 = 4 };

template <int KV>
__host__ __device__ constexpr int kv_bits() {
  return KV == kKvF32 ? 32 : KV == kKvF16 ? 16 : KV == kKvInt4 ? 4 : 8;
}
__host__ __device__ constexpr int cmin(int a, int b) { return a < b ? a : b; }

// BYTES (2, 4, 8 or 16) of a cache row into words; the address is a multiple of BYTES.
template <int BYTES>
__device__ __forceinline__ void load_raw(const unsigned char* p, uint32_t (&w)[4]) {
  if (BYTES == 16) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = x.x, w[1] = x.y, w[2] = x.z, w[3] = x.w;
  } else if (BYTES == 8) {
    const uint2 x = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = x.x, w[1] = x.y;
  } else if (BYTES == 4) {
    w[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
  } else {
    w[0] = __ldg(reinterpret_cast<const unsigned short*>(p));
  }
}

// The N cache elements packed in w, as fp32 (before the key row's scale).
template <int KV, int N>
__device__ __forceinline__ void decode(const uint32_t (&w)[4], float (&out)[N]) {
  if constexpr (KV == kKvFp8) {  // two bytes per conversion (every E4M3 value is exact in binary16)
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((w[i / 4] >> (16 * ((i / 2) % 2))) & 0xFFFFu), __NV_E4M3);
      const float2 f = __half22float2(__half2(h));
      out[i] = f.x, out[i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (KV == kKvF32) {
        out[i] = __uint_as_float(w[i]);
      } else if (KV == kKvF16) {
        out[i] = fp16_bits_to_float((w[i / 2] >> (16 * (i % 2))) & 0xFFFFu);
      } else if (KV == kKvInt8) {
        out[i] = static_cast<float>(static_cast<signed char>((w[i / 4] >> (8 * (i % 4))) & 0xFFu));
      } else {
        // two's-complement nibble i: bits 4 (i % 2) of byte i / 2
        out[i] = static_cast<float>(static_cast<int>(w[i / 8] << (28 - 4 * (i % 8))) >> 28);
      }
    }
  }
}

struct AttnParams {
  const float* q;
  const void* k;
  const void* v;
  const float* ks;
  const float* vs;
  // partial of (query row i, head h, chunk s) at base = (i * heads + h) * splits + s: pacc[base * head_dim ..],
  // pmax[base], psum[base]; an empty chunk is the null partial (0, kNullMax, 0)
  // (the layout of the reference's split kernels, src/backends/rocm/rocm_kernels_basic.cpp:278-330)
  float* pacc;
  float* pmax;
  float* psum;
  int m, n, heads, kv_heads, head_dim, window, causal, splits;
  unsigned long long q_base, row_base;
};

constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
constexpr float kNoKey = -3.0e38f;  // score of a key outside the chunk, and the running max before the first key

// One CTA: one query row, one kv head (all G query heads of its group), one chunk of the key range.
// Scores: 8 lanes share a key (each 1/8 of head_dim in 16-byte pieces, a row read as contiguous 128-byte
// lines), 4 keys per warp and trip, q from shared memory (scaled by log2(e) / sqrt(head_dim), stored so
// that the 8 lanes' pieces lie side by side); the 8 partial dot products meet by shuffles.
// Softmax: running max and sum per head in base-2 exponents, the accumulators rescaled only when the max
// of a trip's keys exceeds it.  Values: the 32 lanes split head_dim, key by key, the key's weight
// broadcast from the lane that holds it.  Scales of a quantised row multiply the score / the weight.
template <int KV, int D, int G>
__global__ void __launch_bounds__(kAttnWarps * 32, 2) attention_chunk_kernel(const AttnParams p) {
  constexpr int BITS = kv_bits<KV>();
  constexpr int EL = D / 8, VEC = cmin(128 / BITS, EL), NV = EL / VEC;  // per lane of a key's 8: NV pieces of VEC elements
  constexpr int EV = D / 32, VV = cmin(128 / BITS, EV), NVV = EV / VV;  // per lane of 32: NVV pieces of VV elements
  constexpr bool kScaled = KV >= kKvFp8;
  extern __shared__ __align__(16) float sh[];
  float* q_s = sh;                           // [G][D], piece (t, u) of the 8 lanes side by side
  float* wmax = q_s + G * D;                 // [warps][G]
  float* wsum = wmax + kAttnWarps * G;       // [warps][G]
  float* part = wsum + kAttnWarps * G;       // [warps][G][D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = lane >> 3, sub = lane & 7;
  const int kv = blockIdx.x / p.splits, split = blockIdx.x - kv * p.splits, i = blockIdx.y;
  const int group = p.heads / p.kv_heads;
  const size_t pos = p.q_base + i;
  const int last = p.causal ? static_cast<int>(pos >= static_cast<size_t>(p.n) ? p.n - 1 : pos) : p.n - 1;
  int start = 0;
  if (p.causal) {
    start = (p.window != 0 && pos + 1 > static_cast<size_t>(p.window)) ? static_cast<int>(pos + 1 - p.window) : 0;
    if (start > last) start = last;
  }
  const int keys = last - start + 1, chunk = (keys + p.splits - 1) / p.splits;
  const int c0 = start + split * chunk, c1 = min(last + 1, c0 + chunk);
  const size_t part0 = (static_cast<size_t>(i) * p.heads + kv * group) * p.splits + split;  // head g: + g * splits
  if (c0 >= c1) {  // the whole CTA: null partials
    for (int t = threadIdx.x; t < group * D; t += blockDim.x) {
      const int g = t / D;
      p.pacc[(part0 + static_cast<size_t>(g) * p.splits) * D + (t - g * D)] = 0.0f;
    }
    if (threadIdx.x < group) {
      p.pmax[part0 + static_cast<size_t>(threadIdx.x) * p.splits] = kNullMax;
      p.psum[part0 + static_cast<size_t>(threadIdx.x) * p.splits] = 0.0f;
    }
    return;
  }
  // The first trip's loads are issued before q is staged.  With 16-bit and narrower caches the later trips' are
  // issued a phase early (a trip's keys while the trip before it does its softmax and values, its values while
  // the next scores are formed); the fp32 cache's words need the registers, so its trips load at their start
  // (measured: 18.3 against 19.8 us per layer at 4096 keys).
  constexpr bool kEarly = BITS <= 16;
  const size_t row_bytes = static_cast<size_t>(p.kv_heads) * D * BITS / 8;
  const unsigned char* kbase = static_cast<const unsigned char*>(p.k) + static_cast<size_t>(kv) * D * BITS / 8;
  const unsigned char* vbase = static_cast<const unsigned char*>(p.v) + static_cast<size_t>(kv) * D * BITS / 8;
  uint32_t kraw[NV][4], vraw[4][NVV][4];
  float kscale = 1.0f, vscale = 1.0f;
  auto load_keys = [&](int base) {
    const int j = min(base + grp, c1 - 1);
#pragma unroll
    for (int t = 0; t < NV; ++t)
      load_raw<VEC * BITS / 8>(kbase + j * row_bytes + (t * 8 * VEC + sub * VEC) * BITS / 8, kraw[t]);
    if (kScaled) kscale = __ldg(p.ks + j), vscale = __ldg(p.vs + j);
  };
  auto load_values = [&](int base) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int jj = min(base + kk, c1 - 1);
#pragma unroll
      for (int t = 0; t < NVV; ++t)
        load_raw<VV * BITS / 8>(vbase + jj * row_bytes + (t * 32 * VV + lane * VV) * BITS / 8, vraw[kk][t]);
    }
  };
  const int first = c0 + warp * 4;
  if (first < c1) {
    load_keys(first);
    load_values(first);
  }
  {
    const float qscale = kLog2e / sqrtf(static_cast<float>(D));
    const float* qrow = p.q + ((p.row_base + i) * p.heads + static_cast<size_t>(kv) * group) * D;
    for (int t = threadIdx.x; t < G * D; t += blockDim.x) {
      const int g = t / D, e = t - g * D;
      // element e = piece * (8 VEC) + sub * VEC + 4 u + c  ->  ((piece * (VEC / 4) + u) * 8 + sub) * 4 + c
      const int piece = e / (8 * VEC), r = e - piece * (8 * VEC), sb = r / VEC, r2 = r - sb * VEC, u = r2 >> 2, c = r2 & 3;
      q_s[g * D + ((piece * (VEC / 4) + u) * 8 + sb) * 4 + c] = g < group ? qrow[t] * qscale : 0.0f;
    }
  }
  __syncthreads();

  float mx[G], sm[G], acc[G][EV];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = kNoKey;
    sm[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < EV; ++e) acc[g][e] = 0.0f;
  }
  for (int base = first; base < c1; base += kAttnWarps * 4) {
    const bool valid = base + grp < c1;
    const int next = base + kAttnWarps * 4;
    if (!kEarly && base != first) {
      load_keys(base);
      load_values(base);
    }
    const float kscale_now = kscale, vscale_now = vscale;  // of this trip's key, before the next trip's loads
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.0f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      float kx[VEC];
      decode<KV, VEC>(kraw[t], kx);
#pragma unroll
      for (int u = 0; u < VEC / 4; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qq = *reinterpret_cast<const float4*>(q_s + g * D + ((t * (VEC / 4) + u) * 8 + sub) * 4);
          s[g] = fmaf(qq.x, kx[4 * u], s[g]);
          s[g] = fmaf(qq.y, kx[4 * u + 1], s[g]);
          s[g] = fmaf(qq.z, kx[4 * u + 2], s[g]);
          s[g] = fmaf(qq.w, kx[4 * u + 3], s[g]);
        }
    }
    if (kEarly && next < c1) load_keys(next);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1)
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xFFFFFFFFu, s[g], o);
    float w[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sc = valid ? s[g] * kscale_now : kNoKey;
      float top = fmaxf(sc, __shfl_xor_sync(0xFFFFFFFFu, sc, 8));
      top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, 16));
      if (top > mx[g]) {  // the same in every lane
        const float corr = exp2f(mx[g] - top);
        sm[g] *= corr;
#pragma unroll
        for (int e = 0; e < EV; ++e) acc[g][e] *= corr;
        mx[g] = top;
      }
      const float wk = exp2f(sc - mx[g]);
      sm[g] += wk;  // this lane's keys; its 8 lanes hold the same sum
      w[g] = wk * vscale_now;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      if (base + kk < c1) {
        float vx[EV];
#pragma unroll
        for (int t = 0; t < NVV; ++t) {
          float piece[VV];
          decode<KV, VV>(vraw[kk][t], piece);
#pragma unroll
          for (int c = 0; c < VV; ++c) vx[t * VV + c] = piece[c];
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float wk = __shfl_sync(0xFFFFFFFFu, w[g], kk * 8);
#pragma unroll
          for (int e = 0; e < EV; ++e) acc[g][e] = fmaf(wk, vx[e], acc[g][e]);
        }
      }
    }
    if (kEarly && next < c1) load_values(next);
  }
  // the warps meet: the CTA's max per head, every warp's share rescaled to it, summed in warp order
#pragma unroll
  for (int g = 0; g < G; ++g) {
    sm[g] += __shfl_xor_sync(0xFFFFFFFFu, sm[g], 8);
    sm[g] += __shfl_xor_sync(0xFFFFFFFFu, sm[g], 16);
    if (lane == 0) wmax[warp * G + g] = mx[g];
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float top = wmax[g];
    for (int wi = 1; wi < kAttnWarps; ++wi) top = fmaxf(top, wmax[wi * G + g]);
    const float f = exp2f(mx[g] - top);  // 0 for a warp that had no key
    if (lane == 0) wsum[warp * G + g] = sm[g] * f;
#pragma unroll
    for (int t = 0; t < NVV; ++t)
#pragma unroll
      for (int c = 0; c < VV; ++c) part[(warp * G + g) * D + t * 32 * VV + lane * VV + c] = acc[g][t * VV + c] * f;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < group * D; t += blockDim.x) {
    const int g = t / D;
    float total = 0.0f;
#pragma unroll
    for (int wi = 0; wi < kAttnWarps; ++wi) total += part[wi * G * D + t];
    p.pacc[(part0 + static_cast<size_t>(g) * p.splits) * D + (t - g * D)] = total;
  }
  if (threadIdx.x < group) {
    const int g = threadIdx.x;
    float top = wmax[g], total = 0.0f;
    for (int wi = 1; wi < kAttnWarps; ++wi) top = fmaxf(top, wmax[wi * G + g]);
    for (int wi = 0; wi < kAttnWarps; ++wi) total += wsum[wi * G + g];
    p.pmax[part0 + static_cast<size_t>(g) * p.splits] = top * kLn2;  // back to a natural-log exponent
    p.psum[part0 + static_cast<size_t>(g) * p.splits] = total;
  }
}

// "attention_combine" (src/backends/rocm/rocm_kernels_basic.cpp:664-686 of the reference):
// out[row][head][e] = sum_s w_s pacc_s[e] / sum_s w_s psum_s, w_s = exp(pmax_s - max_s pmax_s), chunks in order.
// One CTA merges 64 output elements of one (row, head): four quarter-CTAs each take every fourth chunk and
// have their partial values in flight (up to 16 each) while warp 0 finds the max and the denominator; the
// quarters meet in order.
__global__ void __launch_bounds__(256)
attention_combine_kernel(const float* __restrict__ pacc, const float* __restrict__ pmax, const float* __restrict__ psum,
                         float* __restrict__ out, const float* __restrict__ gate, int heads, int head_dim, int splits,
                         unsigned long long row_base) {
  constexpr int kHeld = 16;   // chunks a thread holds in registers: 4 * 16 = 64 chunks without a second round of loads
  __shared__ float w_s[256];  // the weights of the first 256 chunks, computed once
  __shared__ float quarter[4][64];
  __shared__ float top_s, den_s;
  const size_t g = blockIdx.x, base = g * splits;
  const size_t i = g / heads, h = g - i * heads;
  const int lane = threadIdx.x & 31;
  const int col = threadIdx.x & 63, e = blockIdx.y * 64 + col, part = threadIdx.x >> 6;
  float held[kHeld];
#pragma unroll
  for (int r = 0; r < kHeld; ++r) {
    const int s = part + 4 * r;
    held[r] = (s < splits && e < head_dim) ? pacc[(base + s) * head_dim + e] : 0.0f;
  }
  if (threadIdx.x < 32) {
    float top = kNullMax;
    for (int s = lane; s < splits; s += 32) top = fmaxf(top, pmax[base + s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
    float den = 0.0f;
    for (int s = lane; s < splits; s += 32) {
      const float w = expf(pmax[base + s] - top);
      if (s < 256) w_s[s] = w;
      den = fmaf(w, psum[base + s], den);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, o);
    if (lane == 0) top_s = top, den_s = den;
  }
  __syncthreads();
  float num = 0.0f;
  if (e < head_dim) {
    const float top = top_s;
#pragma unroll
    for (int r = 0; r < kHeld; ++r) {
      const int s = part + 4 * r;
      if (s < splits) num = fmaf(w_s[s], held[r], num);
    }
    for (int s = part + 4 * kHeld; s < splits; s += 4) {
      const float w = s < 256 ? w_s[s] : expf(pmax[base + s] - top);
      num = fmaf(w, pacc[(base + s) * head_dim + e], num);
    }
  }
  quarter[part][col] = num;
  __syncthreads();
  if (part == 0 && e < head_dim) {
    const size_t at = ((row_base + i) * heads + h) * head_dim + e;
    const float v = (((quarter[0][col] + quarter[1][col]) + quarter[2][col]) + quarter[3][col]) / den_s;
    // the sigmoid_gate step that follows attention in the reference's layer, when the queue merged it in
    out[at] = gate != nullptr ? v / (1.0f + expf(-gate[at])) : v;
  }
}

template <int KV, int D, int G>
int launch_chunks_g(const AttnParams& p, cudaStream_t st) {
  const size_t smem = (static_cast<size_t>(G) * D * (1 + kAttnWarps) + 2 * kAttnWarps * G) * sizeof(float);
  static bool raised[64] = {};  // per device: the kernel may use more than the default 48 KB of shared memory
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kDeviceError;
  if (!raised[dev]) {
    if (cudaFuncSetAttribute(attention_chunk_kernel<KV, D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return kDeviceError;
    raised[dev] = true;
  }
  const dim3 grid(static_cast<unsigned>(p.kv_heads * p.splits), static_cast<unsigned>(p.m));
  attention_chunk_kernel<KV, D, G><<<grid, kAttnWarps * 32, smem, st>>>(p);
  return check_launch();
}

template <int KV, int D>
int launch_chunks_d(const AttnParams& p, cudaStream_t st) {
  const int group = p.heads / p.kv_heads;
  if (group <= 2) return launch_chunks_g<KV, D, 2>(p, st);
  if (group <= 4) return launch_chunks_g<KV, D, 4>(p, st);
  if (group <= 6) return launch_chunks_g<KV, D, 6>(p, st);
  return launch_chunks_g<KV, D, 8>(p, st);
}

template <int KV>
int launch_split(const AttnParams& p, cudaStream_t st) {
  return p.head_dim == 256 ? launch_chunks_d<KV, 256>(p, st) : launch_chunks_d<KV, 128>(p, st);
}

int run_split(int kvkind, const AttnParams& p, cudaStream_t st) {
  switch (kvkind) {
    case kKvF32: return launch_split<kKvF32>(p, st);
    case kKvF16: return launch_split<kKvF16>(p, st);
    case kKvFp8: return launch_split<kKvFp8>(p, st);
    case kKvInt4: return launch_split<kKvInt4>(p, st);
    default: return launch_split<kKvInt8>(p, st);
  }
}

int run_combine(const float* pacc, const float* pmax, const float* psum, float* out, const float* gate, uint64_t m,
                uint64_t heads, uint64_t head_dim, uint64_t splits, uint64_t row_base, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>(m * heads), static_cast<unsigned>((head_dim + 63) / 64));
  attention_combine_kernel<<<grid, 256, 0, st>>>(pacc, pmax, psum, out, gate, static_cast<int>(heads), static_cast<int>(head_dim),
                                                 static_cast<int>(splits), row_base);
  return check_launch();
}

// Argument checks shared by the entry points; fills the kernel's parameters except the partial buffers.
int check_attention(int kvkind, const float* q, const void* k, const void* v, const float* ks, const float* vs, uint64_t m,
                    uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim, uint64_t q_base, uint64_t row_base,
                    uint64_t window, uint64_t causal, uint64_t splits, AttnParams* p) {
  if (!q || !k || !v || m == 0 || n == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || heads % kv_heads != 0 ||
      m > 65535 || n > 0x7FFFFFFFull || heads > 65535 || window > 0x7FFFFFFFull || splits == 0 || splits > 64)
    return kInvalidArgument;
  if (kvkind >= kKvFp8 && (!ks || !vs)) return kInvalidArgument;
  if ((head_dim != 128 && head_dim != 256) || heads / kv_heads > kAttnMaxGroup) return kUnsupportedFeature;
  *p = AttnParams{q, k, v, ks, vs, nullptr, nullptr, nullptr, static_cast<int>(m), static_cast<int>(n),
                  static_cast<int>(heads), static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(window),
                  causal != 0 ? 1 : 0, static_cast<int>(splits), q_base, row_base};
  return kOk;
}

int run_attention(int kvkind, const float* q, const void* k, const void* v, const float* ks, const float* vs, float* out,
                  const float* gate, uint64_t m, uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim,
                  uint64_t q_base, uint64_t row_base, uint64_t window, uint64_t causal, cudaStream_t st) {
  if (!out) return kInvalidArgument;
  // as many chunks as keep a CTA busy with kAttnMinKeys keys, counted on the longest row's range
  const uint64_t span = window != 0 && window < n ? window : n;
  uint64_t splits = span / kAttnMinKeys;
  if (splits < 1) splits = 1;
  if (splits > kAttnMaxSplits) splits = kAttnMaxSplits;
  AttnParams p;
  if (int rc = check_attention(kvkind, q, k, v, ks, vs, m, n, heads, kv_heads, head_dim, q_base, row_base, window, causal,
                               splits, &p))
    return rc;
  const size_t parts = m * heads * splits;
  const size_t acc_bytes = parts * head_dim * 4, stat_bytes = (parts * 4 + 255) / 256 * 256;
  unsigned char* scratch = stream_scratch(st, acc_bytes + 2 * stat_bytes, 2);
  if (scratch == nullptr) return kUnsupportedFeature;
  p.pacc = reinterpret_cast<float*>(scratch);
  p.pmax = reinterpret_cast<float*>(scratch + acc_bytes);
  p.psum = reinterpret_cast<float*>(scratch + acc_bytes + stat_bytes);
  if (int rc = run_split(kvkind, p, st)) return rc;
  return run_combine(p.pacc, p.pmax, p.psum, out, gate, m, heads, head_dim, splits, row_base, st);
}

int kv_kind_of(int kv_format) {
  switch (kv_format) {
    case TSR_KV_F32: return kKvF32;
    case TSR_KV_F16: return kKvF16;
    case TSR_KV_INT8: return kKvInt8;
    case TSR_KV_INT4: return kKvInt4;
    case TSR_KV_FP8: return kKvFp8;
    default: return -1;
  }
}

}  // namespace

int attention_gated(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                    float* out, const float* gate, uint64_t m, uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim,
                    uint64_t q_base, uint64_t row_base, uint64_t window, uint64_t causal, cudaStream_t st) {
  const int kind = kv_kind_of(kv_format);
  if (kind < 0) return kInvalidArgument;
  return run_attention(kind, q, k, v, k_scale, v_scale, out, gate, m, n, heads, kv_heads, head_dim, q_base, row_base, window,
                       causal, st);
}
}  // namespace tsr

using namespace tsr;

extern "C" {

int tsr_attention(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                  float* out, uint64_t m, uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim, uint64_t q_base,
                  uint64_t row_base, uint64_t window, uint64_t causal, void* stream) {
  return attention_gated(kv_format, q, k, v, k_scale, v_scale, out, nullptr, m, n, heads, kv_heads, head_dim, q_base, row_base,
                         window, causal, static_cast<cudaStream_t>(stream));
}

int tsr_attention_split(int kv_format, const float* q, const void* k, const void* v, const float* k_scale,
                        const float* v_scale, float* pacc, float* pmax, float* psum, uint64_t m, uint64_t n, uint64_t heads,
                        uint64_t kv_heads, uint64_t head_dim, uint64_t q_base, uint64_t window, uint64_t causal, uint64_t split,
                        void* stream) {
  const int kind = kv_kind_of(kv_format);
  if (kind < 0 || !pacc || !pmax || !psum) return kInvalidArgument;
  AttnParams p;
  if (int rc = check_attention(kind, q, k, v, k_scale, v_scale, m, n, heads, kv_heads, head_dim, q_base, 0, window, causal,
                               split, &p))
    return rc;
  p.pacc = pacc, p.pmax = pmax, p.psum = psum;
  return run_split(kind, p, static_cast<cudaStream_t>(stream));
}

int tsr_attention_combine(const float* pacc, const float* pmax, const float* psum, float* out, uint64_t m, uint64_t heads,
                          uint64_t head_dim, uint64_t split, void* stream) {
  if (!pacc || !pmax || !psum || !out || m == 0 || heads == 0 || head_dim == 0 || split == 0 || m * heads > 0x7FFFFFFFull ||
      split > 0x7FFFFFFFull || head_dim > 0x7FFFFFFFull)
    return kInvalidArgument;
  return run_combine(pacc, pmax, psum, out, nullptr, m, heads, head_dim, split, 0, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
