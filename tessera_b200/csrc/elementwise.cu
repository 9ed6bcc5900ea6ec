// Small kernels around the projections: per-token FP8 activation
// quantisation, split-K reduce, bf16 rounding, add, fill, the MXFP4 row
// reference byte, and the bit-exact block dequantiser used by the codec
// parity tests.
#include "codec.cuh"
#include "launch.h"
#include "tessera_b200.h"

namespace tsr {

// ------------------------------------------------ per-token FP8 quantise
// One CTA per row.  scale = max(amax/448, 1/(448*512)); q = clamp(x/scale,
// +-448) coded to E4M3 round-to-nearest-even
// (src/core/numerics/quant.cpp:180-229).  PACK writes codes, else the data is
// replaced by code*scale in place.
template <bool PACK>
__global__ void __launch_bounds__(1024)
quantize_fp8_kernel(float* __restrict__ data, const float* __restrict__ in,
                    uint8_t* __restrict__ codes, float* __restrict__ scale, int cols) {
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * cols;
  const float* src = PACK ? in + base : data + base;
  float amax = 0.0f;
  for (int cidx = threadIdx.x; cidx < cols; cidx += blockDim.x)
    amax = fmaxf(amax, fabsf(src[cidx]));  // fmaxf drops NaN like std::max(amax, x)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float s = fmaxf(__fdiv_rn(red[0], 448.0f), 1.0f / (448.0f * 512.0f));
  if (threadIdx.x == 0) scale[blockIdx.x] = s;
  for (int cidx = threadIdx.x; cidx < cols; cidx += blockDim.x) {
    float q = __fdiv_rn(src[cidx], s);
    q = q < -448.0f ? -448.0f : (448.0f < q ? 448.0f : q);  // std::clamp; NaN passes through
    const uint32_t code = float_to_e4m3_ref(q);
    if (PACK) {
      codes[base + cidx] = static_cast<uint8_t>(code);
    } else {
      data[base + cidx] = __fmul_rn(e4m3_to_float(code), s);
    }
  }
}

// gemm_vec_reduce.comp:20-32: ordered sum of the split regions.
__global__ void vec_reduce_kernel(const float* __restrict__ part, float* __restrict__ c,
                                  size_t total, int split) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  pdl_wait();     // the partials come from the kernel just ahead
  pdl_trigger();  // the next projection may start prefetching its weights
  if (i >= total) return;
  float acc = 0.0f;
  for (int s = 0; s < split; ++s) acc += part[s * total + i];
  c[i] = acc;
}

// round_bf16.comp:14-24 / quant.cpp:231-243.
__global__ void round_bf16_kernel(float* __restrict__ x, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t u = __float_as_uint(x[i]);
  u += 0x7FFFu + ((u >> 16) & 1u);
  x[i] = __uint_as_float(u & 0xFFFF0000u);
}

__global__ void bf16_to_f32_kernel(const unsigned short* __restrict__ src, float* __restrict__ dst, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __uint_as_float(static_cast<uint32_t>(src[i]) << 16);
}

// the rounding of round_bf16_kernel, stored as the high half
__global__ void f32_to_bf16_kernel(const float* __restrict__ src, unsigned short* __restrict__ dst, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t u = __float_as_uint(src[i]);
  u += 0x7FFFu + ((u >> 16) & 1u);
  dst[i] = static_cast<unsigned short>(u >> 16);
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                           float* __restrict__ o, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) o[i] = a[i] + b[i];
}

__global__ void fill_kernel(int32_t* __restrict__ d, int32_t v, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) d[i] = v;
}

// mxfp4_row_ref.comp:26-40: largest E8M0 byte of each row; warp per row.
__global__ void mxfp4_row_ref_kernel(const uint8_t* __restrict__ w, uint8_t* __restrict__ wref,
                                     int n, int k) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n) return;
  const int nb = k / 32;
  const uint8_t* s = w + static_cast<size_t>(n) * (k / 2) + static_cast<size_t>(row) * nb;
  uint32_t mx = 0;
  for (int b = threadIdx.x & 31; b < nb; b += 32) mx = max(mx, static_cast<uint32_t>(s[b]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  if ((threadIdx.x & 31) == 0) wref[row] = static_cast<uint8_t>(mx);
}

// Bit-exact dequantiser: one thread per element, every product and the
// subtraction rounded separately, as the host reference does without fused
// multiply-add.
__global__ void dequantize_kernel(int fmt, const uint8_t* __restrict__ w,
                                  const float* __restrict__ row_scale, float* __restrict__ out,
                                  size_t n, size_t k) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n * k) return;
  const size_t row = idx / k, t = idx % k;
  float v = 0.0f;
  if (fmt == 0) {
    const uint8_t* blk = w + (row * (k / 256) + t / 256) * kQ4KBlockBytes;
    const int e = static_cast<int>(t % 256), g = e / 64, hi = (e % 64) / 32, l = e % 32;
    const float d = fp16_bits_to_float(blk[0] | (blk[1] << 8));
    const float dmin = fp16_bits_to_float(blk[2] | (blk[3] << 8));
    uint32_t s[3];
    for (int i = 0; i < 3; ++i)
      s[i] = blk[4 + 4 * i] | (blk[5 + 4 * i] << 8) | (blk[6 + 4 * i] << 16) |
             (static_cast<uint32_t>(blk[7 + 4 * i]) << 24);
    uint32_t sc, mn;
    q4k_scale_min(s, 2 * g + hi, sc, mn);
    const uint32_t byte = blk[16 + 32 * g + l];
    const float q = static_cast<float>(hi ? (byte >> 4) : (byte & 15u));
    v = __fsub_rn(__fmul_rn(__fmul_rn(d, static_cast<float>(sc)), q),
                  __fmul_rn(dmin, static_cast<float>(mn)));
  } else if (fmt == 1) {
    const uint8_t* blk = w + (row * (k / 256) + t / 256) * kQ6KBlockBytes;
    const int e = static_cast<int>(t % 256), h = e / 128, part = (e % 128) / 32, l = e % 32;
    const float d = fp16_bits_to_float(blk[208] | (blk[209] << 8));
    const uint32_t lo = blk[64 * h + 32 * (part & 1) + l];
    const uint32_t qh = blk[128 + 32 * h + l];
    const uint32_t nib = (part & 2) ? (lo >> 4) : (lo & 15u);
    const int q = static_cast<int>(nib | (((qh >> (2 * part)) & 3u) << 4)) - 32;
    const float sc = static_cast<float>(static_cast<signed char>(blk[192 + 8 * h + l / 16 + 2 * part]));
    v = __fmul_rn(__fmul_rn(d, sc), static_cast<float>(q));
  } else if (fmt == 2) {
    const uint32_t byte = w[(row * k + t) / 2];
    const uint32_t nib = (t % 2 == 0) ? (byte & 15u) : (byte >> 4);
    const uint32_t sb = w[n * (k / 2) + row * (k / 32) + t / 32];
    v = __fmul_rn(e8m0_to_float(sb), e2m1_to_float(nib));
  } else {
    v = __fmul_rn(row_scale[row], e4m3_to_float(w[row * k + t]));
  }
  out[idx] = v;
}

// O = silu(G) * U (SiluMulRef, src/core/numerics/norm.cpp:211-225)
__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ o,
                                size_t n) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const float x = g[idx];
  o[idx] = x / (1.0f + expf(-x)) * u[idx];
}

// Y = X / sqrt(mean(X^2) + eps) * W, one CTA per row (RmsNormRef, src/core/numerics/norm.cpp:7-32;
// the reference adds the squares sequentially, here they are added as a tree).
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int cols, float eps) {
  __shared__ float red[32];
  const float* row = x + static_cast<size_t>(blockIdx.x) * cols;
  float s = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s = fmaf(row[c], row[c], s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / static_cast<float>(cols) + eps);
  }
  __syncthreads();
  const float gain = red[0];
  float* out = y + static_cast<size_t>(blockIdx.x) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) out[c] = row[c] * gain * w[c];
}

static unsigned blocks_for(uint64_t n, unsigned per) {
  return static_cast<unsigned>((n + per - 1) / per);
}

int convert_bf16_to_f32(const void* src, float* dst, uint64_t n, cudaStream_t st) {
  bf16_to_f32_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<const unsigned short*>(src), dst, n);
  return check_launch();
}
int convert_f32_to_bf16(const float* src, void* dst, uint64_t n, cudaStream_t st) {
  f32_to_bf16_kernel<<<blocks_for(n, 256), 256, 0, st>>>(src, static_cast<unsigned short*>(dst), n);
  return check_launch();
}

}  // namespace tsr

using namespace tsr;

extern "C" {

int tsr_quantize_fp8(float* data, float* scale, uint64_t rows, uint64_t cols, void* stream) {
  if (!data || !scale || rows == 0 || cols == 0 || cols > 0x7FFFFFFFull) return kInvalidArgument;
  quantize_fp8_kernel<false><<<static_cast<unsigned>(rows), 1024, 0,
                               static_cast<cudaStream_t>(stream)>>>(data, nullptr, nullptr, scale,
                                                                    static_cast<int>(cols));
  return check_launch();
}

int tsr_quantize_fp8_pack(const float* in, void* out, float* scale, uint64_t rows, uint64_t cols,
                          void* stream) {
  if (!in || !out || !scale || rows == 0 || cols == 0 || cols % 4 != 0 || cols > 0x7FFFFFFFull)
    return kInvalidArgument;
  quantize_fp8_kernel<true><<<static_cast<unsigned>(rows), 1024, 0,
                              static_cast<cudaStream_t>(stream)>>>(
      nullptr, in, static_cast<uint8_t*>(out), scale, static_cast<int>(cols));
  return check_launch();
}

int tsr_gemm_vec_reduce(const float* part, float* c, uint64_t total, uint64_t split, void* stream) {
  if (!part || !c || total == 0 || split == 0) return kInvalidArgument;
  auto st = static_cast<cudaStream_t>(stream);
  // reads the partial buffer only after its wait, so it can always be a programmatic dependent
  const bool pdl = pdl_allowed(st, nullptr, 0, c, total * 4);
  launch_kernel(vec_reduce_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, st, pdl, part, c,
                static_cast<size_t>(total), static_cast<int>(split));
  return check_launch();
}

int tsr_round_bf16(float* x, uint64_t n, void* stream) {
  if (!x || n == 0) return kInvalidArgument;
  round_bf16_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, n);
  return check_launch();
}

int tsr_add(const float* a, const float* b, float* o, uint64_t n, void* stream) {
  if (!a || !b || !o || n == 0) return kInvalidArgument;
  add_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b, o, n);
  return check_launch();
}

int tsr_silu_mul(const float* g, const float* u, float* o, uint64_t n, void* stream) {
  if (!g || !u || !o || n == 0) return kInvalidArgument;
  silu_mul_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(g, u, o, n);
  return check_launch();
}

int tsr_rmsnorm(const float* x, const float* w, float* y, uint64_t rows, uint64_t cols, float eps, void* stream) {
  if (!x || !w || !y || rows == 0 || cols == 0 || rows > 0x7FFFFFFFull || cols > 0x7FFFFFFFull || !(eps >= 0.0f))
    return kInvalidArgument;
  rmsnorm_kernel<<<static_cast<unsigned>(rows), cols >= 4096 ? 1024 : 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, w, y, static_cast<int>(cols), eps);
  return check_launch();
}

int tsr_fill(int32_t* data, int32_t value, uint64_t n, void* stream) {
  if (!data || n == 0) return kInvalidArgument;
  fill_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(data, value, n);
  return check_launch();
}

int tsr_mxfp4_row_ref(const void* w, void* wref, uint64_t n, uint64_t k, void* stream) {
  if (!w || !wref || n == 0 || k == 0 || k % 32 != 0) return kInvalidArgument;
  mxfp4_row_ref_kernel<<<blocks_for(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(w), static_cast<uint8_t*>(wref), static_cast<int>(n),
      static_cast<int>(k));
  return check_launch();
}

int tsr_dequantize(int fmt, const void* w, const float* row_scale, float* out, uint64_t n,
                   uint64_t k, void* stream) {
  if (!w || !out || n == 0 || k == 0 || fmt < 0 || fmt > 3) return kInvalidArgument;
  if ((fmt <= 1 && k % 256 != 0) || (fmt == 2 && k % 32 != 0) || (fmt == 3 && !row_scale))
    return kInvalidArgument;
  dequantize_kernel<<<blocks_for(n * k, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      fmt, static_cast<const uint8_t*>(w), row_scale, out, n, k);
  return check_launch();
}

}  // extern "C"
