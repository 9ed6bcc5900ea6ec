/*
 * CPU oracle for the quantized projection path (see oracle.h).
 * TEST INFRASTRUCTURE ONLY.  Plain C restatement of the reference's host
 * reference functions; compiled with -ffp-contract=off so that the only
 * fused operations are the explicit fmaf() calls the reference also makes.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ codecs */

static float bits_to_float(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint32_t float_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* IEEE binary16 -> binary32.  quant.cpp:75-93 */
float orc_fp16_to_float(uint16_t h) {
  uint32_t e = (h >> 10) & 31u, m = h & 1023u;
  float v;
  if (e == 0) {
    v = (float)m * 0x1p-24f;
  } else if (e == 31) {
    v = m ? nanf("") : INFINITY;
  } else {
    v = (1.0f + (float)m / 1024.0f) * ldexpf(1.0f, (int)e - 15);
  }
  return (h & 0x8000u) ? -v : v;
}

/* quant.cpp:95-100 */
float orc_bf16_to_float(uint16_t b) { return bits_to_float((uint32_t)b << 16); }

/* Truncating binary32 -> binary16 used by the reference's cast helper.
 * quant.cpp:102-124 */
uint16_t orc_fp16_from_float(float v) {
  uint32_t u = float_to_bits(v);
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t e = (int32_t)((u >> 23) & 0xFF) - 127;
  uint32_t man = u & 0x7FFFFFu;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e < -24) return (uint16_t)sign;
  if (e < -14) {
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(-e - 14);
    return (uint16_t)(sign | (man >> (shift + 13)));
  }
  return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | (man >> 13));
}

/* OCP FP8 E4M3 (bias 7, 0x7F/0xFF NaN, max 448).  quant.cpp:258-277 */
float orc_fp8e4m3_to_float(uint8_t b) {
  uint32_t e = (b >> 3) & 15u, m = b & 7u;
  float v;
  if (e == 0) {
    v = (float)m * 0x1p-9f;
  } else if (e == 15) {
    if (m == 7) return nanf("");
    v = (1.0f + (float)m / 8.0f) * 256.0f;
  } else {
    v = (1.0f + (float)m / 8.0f) * ldexpf(1.0f, (int)e - 7);
  }
  return (b & 0x80u) ? -v : v;
}

/* quant.cpp:279-281 */
float orc_e8m0_to_float(uint8_t s) { return ldexpf(1.0f, (int)s - 127); }

/* OCP MX E2M1: {0,.5,1,1.5,2,3,4,6} with sign bit 3.  quant.cpp:283-297 */
float orc_f4e2m1_to_float(uint8_t nib) {
  uint32_t e = (nib >> 1) & 3u, m = nib & 1u;
  float v = (e == 0) ? (float)m * 0.5f
                     : (1.0f + (float)m / 2.0f) * ldexpf(1.0f, (int)e - 1);
  return (nib & 8u) ? -v : v;
}

/* binary32 -> E4M3 byte, round to nearest even, NaN and |v|>448 give the
 * all-ones code; subnormal rounding clamps the mantissa at 7 instead of
 * carrying into the first normal.  quant.cpp:299-342 */
uint8_t orc_fp32_to_fp8e4m3(float v) {
  uint32_t u = float_to_bits(v);
  uint32_t sign = u >> 31;
  if ((u & 0x7FFFFFFFu) > 0x7F800000u || !(v == v)) return (uint8_t)((sign << 7) | 0x7F);
  float mag = v < 0 ? -v : v;
  if (mag == 0.0f) return (uint8_t)(sign << 7);
  if (mag > 448.0f) return (uint8_t)((sign << 7) | 0x7F);
  int ex = 0;
  float fr = frexpf(mag, &ex); /* mag = fr * 2^ex, fr in [0.5,1) */
  int field = ex + 6;
  long long man;
  if (field < 1) {
    man = llrintf(mag * 512.0f);
    if (man > 7) man = 7;
    return (uint8_t)((sign << 7) | (uint32_t)man);
  }
  man = llrintf((fr * 2.0f - 1.0f) * 8.0f);
  if (man == 8) {
    man = 0;
    ++field;
  }
  if (field > 15) field = 15;
  if (field == 15 && man > 6) man = 6;
  return (uint8_t)((sign << 7) | ((uint32_t)field << 3) | (uint32_t)man);
}

/* Nearest E2M1 grid point, first-best on ties, NaN -> 0.  quant.cpp:344-386 */
uint8_t orc_fp32_to_f4e2m1(float v) {
  static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  if (!(v == v)) return 0;
  float mag = v < 0 ? -v : v;
  if (mag > 6.0f) mag = 6.0f;
  uint32_t best = 0;
  float best_d = mag;
  for (uint32_t i = 1; i < 8; ++i) {
    float d = mag > grid[i] ? mag - grid[i] : grid[i] - mag;
    if (d < best_d) {
      best_d = d;
      best = i;
    }
  }
  return (uint8_t)((v < 0 ? 8u : 0u) | best); /* code == index: e<<1|m */
}

/* --------------------------------------------------------------- Q4_K/Q6_K */

/* 6-bit (scale, min) of sub-block j from the 12 packed bytes.
 * quant.cpp:58-70 */
static void q4k_scale_min(unsigned j, const uint8_t* p, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = p[j] & 63;
    *mn = p[j + 4] & 63;
  } else {
    *sc = (uint8_t)((p[j + 4] & 15) | ((p[j - 4] >> 6) << 4));
    *mn = (uint8_t)((p[j + 4] >> 4) | ((p[j] >> 6) << 4));
  }
}

static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* quant.cpp:656-675: d,dmin fp16 @0,@2; scales @4..15; nibbles @16..143.
 * value = (d*sc)*q - (dmin*mn), each product and the difference rounded. */
void orc_dequant_q4k_block(const uint8_t* blk, float* out) {
  const float d = orc_fp16_to_float(rd16(blk));
  const float dmin = orc_fp16_to_float(rd16(blk + 2));
  for (unsigned g = 0; g < 4; ++g) {
    uint8_t sc0, mn0, sc1, mn1;
    q4k_scale_min(2 * g, blk + 4, &sc0, &mn0);
    q4k_scale_min(2 * g + 1, blk + 4, &sc1, &mn1);
    const float s0 = d * (float)sc0, o0 = dmin * (float)mn0;
    const float s1 = d * (float)sc1, o1 = dmin * (float)mn1;
    for (unsigned l = 0; l < 32; ++l) {
      const uint8_t q = blk[16 + 32 * g + l];
      out[64 * g + l] = s0 * (float)(q & 15) - o0;
      out[64 * g + 32 + l] = s1 * (float)(q >> 4) - o1;
    }
  }
}

/* quant.cpp:421-449: ql[128] qh[64] int8 scales[16] d fp16@208;
 * value = d * s * (q - 32), left to right. */
void orc_dequant_q6k_block(const uint8_t* blk, float* out) {
  const float d = orc_fp16_to_float(rd16(blk + 208));
  for (unsigned h = 0; h < 2; ++h) {
    const uint8_t* ql = blk + 64 * h;
    const uint8_t* qh = blk + 128 + 32 * h;
    const int8_t* sc = (const int8_t*)(blk + 192 + 8 * h);
    for (unsigned l = 0; l < 32; ++l) {
      const unsigned is = l / 16;
      const int q1 = (ql[l] & 15) | (((qh[l] >> 0) & 3) << 4);
      const int q2 = (ql[32 + l] & 15) | (((qh[l] >> 2) & 3) << 4);
      const int q3 = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4);
      const int q4 = (ql[32 + l] >> 4) | (((qh[l] >> 6) & 3) << 4);
      out[128 * h + l] = d * sc[is + 0] * (q1 - 32);
      out[128 * h + 32 + l] = d * sc[is + 2] * (q2 - 32);
      out[128 * h + 64 + l] = d * sc[is + 4] * (q3 - 32);
      out[128 * h + 96 + l] = d * sc[is + 6] * (q4 - 32);
    }
  }
}

typedef void (*dequant_fn)(const uint8_t*, float*);

static int fmt_layout(int fmt, size_t* bytes, dequant_fn* fn) {
  if (fmt == 0) {
    *bytes = ORC_Q4K_BLOCK_BYTES;
    *fn = orc_dequant_q4k_block;
    return 0;
  }
  if (fmt == 1) {
    *bytes = ORC_Q6K_BLOCK_BYTES;
    *fn = orc_dequant_q6k_block;
    return 0;
  }
  return -1;
}

int orc_dequant_blocks(int fmt, const uint8_t* bytes, size_t nblocks, float* out) {
  size_t bb;
  dequant_fn fn;
  if (fmt_layout(fmt, &bb, &fn)) return -1;
  for (size_t b = 0; b < nblocks; ++b) fn(bytes + b * bb, out + b * 256);
  return 0;
}

/* ------------------------------------------------------------------- GEMMs */

/* One weight row decoded once, then one sequential-fma dot per A row over
 * the block range [b0, b1).  gemm.cpp:18-41 (full range) */
static void block_row_dots(const float* a, const uint8_t* wrow, float* c, size_t m, size_t n,
                           size_t k, size_t j, size_t b0, size_t b1, size_t bb, dequant_fn fn,
                           float* scratch) {
  for (size_t b = b0; b < b1; ++b) fn(wrow + b * bb, scratch + b * 256);
  for (size_t i = 0; i < m; ++i) {
    const float* ar = a + i * k;
    float acc = 0.0f;
    for (size_t t = b0 * 256; t < b1 * 256; ++t) acc = fmaf(ar[t], scratch[t], acc);
    c[i * n + j] = acc;
  }
}

static int gemm_blocks(int fmt, const float* a, const uint8_t* w, float* c, size_t m, size_t n,
                       size_t k, int threads) {
  size_t bb;
  dequant_fn fn;
  if (fmt_layout(fmt, &bb, &fn)) return -1;
  if (m == 0 || n == 0 || k == 0 || k % 256 != 0) return -1;
  const size_t nb = k / 256;
  int failed = 0;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
  {
    float* scratch = (float*)malloc(k * sizeof(float));
    if (!scratch) {
      failed = 1;
    } else {
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
      for (long long j = 0; j < (long long)n; ++j)
        block_row_dots(a, w + (size_t)j * nb * bb, c, m, n, k, (size_t)j, 0, nb, bb, fn, scratch);
      free(scratch);
    }
  }
  (void)threads;
  return failed ? -2 : 0;
}

int orc_gemm_q4k(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k) {
  return gemm_blocks(0, a, w, c, m, n, k, 1);
}
int orc_gemm_q6k(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k) {
  return gemm_blocks(1, a, w, c, m, n, k, 1);
}
int orc_gemm_q4k_mt(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k, int threads) {
  return gemm_blocks(0, a, w, c, m, n, k, threads);
}
int orc_gemm_q6k_mt(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k, int threads) {
  return gemm_blocks(1, a, w, c, m, n, k, threads);
}

/* gemm.cpp:311-344: weight = scale * e2m1(nibble), low nibble first. */
int orc_gemm_mxfp4_mt(const float* a, const uint8_t* w, const uint8_t* s, float* c, size_t m,
                      size_t n, size_t k, int threads) {
  if (m == 0 || n == 0 || k == 0 || k % ORC_MXFP4_BLOCK != 0) return -1;
  const size_t nb = k / ORC_MXFP4_BLOCK;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
  for (long long jj = 0; jj < (long long)n; ++jj) {
    const size_t j = (size_t)jj;
    for (size_t i = 0; i < m; ++i) {
      float acc = 0.0f;
      for (size_t b = 0; b < nb; ++b) {
        const float sc = orc_e8m0_to_float(s[j * nb + b]);
        for (size_t l = 0; l < ORC_MXFP4_BLOCK; ++l) {
          const size_t t = b * ORC_MXFP4_BLOCK + l;
          const uint8_t byte = w[(j * k + t) / 2];
          const uint8_t nib = (t % 2 == 0) ? (byte & 15) : (byte >> 4);
          acc = fmaf(a[i * k + t], sc * orc_f4e2m1_to_float(nib), acc);
        }
      }
      c[i * n + j] = acc;
    }
  }
  (void)threads;
  return 0;
}
int orc_gemm_mxfp4(const float* a, const uint8_t* w, const uint8_t* s, float* c, size_t m, size_t n,
                   size_t k) {
  return orc_gemm_mxfp4_mt(a, w, s, c, m, n, k, 1);
}

/* gemm.cpp:253-277: weight = s[j] * e4m3(W[j,t]) rounded once, then fma. */
int orc_gemm_fp8_mt(const float* a, const uint8_t* w, const float* s, float* c, size_t m, size_t n,
                    size_t k, int threads) {
  if (m == 0 || n == 0 || k == 0) return -1;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
  for (long long jj = 0; jj < (long long)n; ++jj) {
    const size_t j = (size_t)jj;
    for (size_t i = 0; i < m; ++i) {
      float acc = 0.0f;
      for (size_t t = 0; t < k; ++t)
        acc = fmaf(a[i * k + t], s[j] * orc_fp8e4m3_to_float(w[j * k + t]), acc);
      c[i * n + j] = acc;
    }
  }
  (void)threads;
  return 0;
}
int orc_gemm_fp8(const float* a, const uint8_t* w, const float* s, float* c, size_t m, size_t n,
                 size_t k) {
  return orc_gemm_fp8_mt(a, w, s, c, m, n, k, 1);
}

/* ----------------------------------------------------------------- split-K */

/* decode_internal.hpp:866-885: largest divisor of k/256, at most 8, that
 * reaches `target` workgroups of 8 outputs; 1 when already wide enough. */
size_t orc_gemm_vec_split_rule(size_t outputs, size_t k, size_t target) {
  const size_t bx = (outputs + 7) / 8;
  if (bx == 0 || bx >= target) return 1;
  const size_t sb = k / 256;
  size_t split = (target + bx - 1) / bx;
  if (split > 8) split = 8;
  for (; split > 1; --split)
    if (sb % split == 0) return split;
  return 1;
}

/* gemm_q4k_vec.comp:80-103 (and the Q6_K twin): chunk y covers blocks
 * [y*per, (y+1)*per), per = (k/256)/split, and lands in region y of C. */
int orc_gemm_vec_split(int fmt, const float* a, const uint8_t* w, float* part, size_t m, size_t n,
                       size_t k, size_t split) {
  size_t bb;
  dequant_fn fn;
  if (fmt_layout(fmt, &bb, &fn)) return -1;
  if (m == 0 || n == 0 || k == 0 || k % 256 != 0 || split == 0) return -1;
  const size_t nb = k / 256;
  if (nb % split != 0) return -1;
  const size_t per = nb / split;
  float* scratch = (float*)malloc(k * sizeof(float));
  if (!scratch) return -2;
  for (size_t y = 0; y < split; ++y)
    for (size_t j = 0; j < n; ++j)
      block_row_dots(a, w + j * nb * bb, part + y * m * n, m, n, k, j, y * per, (y + 1) * per, bb,
                     fn, scratch);
  free(scratch);
  return 0;
}

/* gemm_vec_reduce.comp:20-32: ordered sum, plain adds. */
int orc_gemm_vec_reduce(const float* part, float* c, size_t total, size_t split) {
  if (total == 0 || split == 0) return -1;
  for (size_t i = 0; i < total; ++i) {
    float acc = 0.0f;
    for (size_t s = 0; s < split; ++s) acc += part[s * total + i];
    c[i] = acc;
  }
  return 0;
}

/* ---------------------------------------------------- activation quantise */

static const float kE4M3Max = 448.0f;
static const float kE4M3MinScale = 1.0f / (448.0f * 512.0f);

static float row_scale(const float* x, size_t cols) {
  float amax = 0.0f;
  for (size_t c = 0; c < cols; ++c) {
    const float v = fabsf(x[c]);
    if (v > amax) amax = v; /* std::max(amax, |x|): NaN never replaces amax */
  }
  const float s = amax / kE4M3Max;
  return s > kE4M3MinScale ? s : kE4M3MinScale;
}

static float clamp448(float q) {
  /* std::clamp(q, -448, 448): q < lo ? lo : (hi < q ? hi : q); NaN passes. */
  if (q < -kE4M3Max) return -kE4M3Max;
  if (kE4M3Max < q) return kE4M3Max;
  return q;
}

/* quant.cpp:180-205: quantise-dequantise in place, scale out. */
int orc_quantize_fp8(float* data, float* scale, size_t rows, size_t cols) {
  if (rows == 0 || cols == 0) return -1;
  for (size_t r = 0; r < rows; ++r) {
    float* x = data + r * cols;
    const float s = row_scale(x, cols);
    scale[r] = s;
    for (size_t c = 0; c < cols; ++c)
      x[c] = orc_fp8e4m3_to_float(orc_fp32_to_fp8e4m3(clamp448(x[c] / s))) * s;
  }
  return 0;
}

/* quant.cpp:207-229: same scale, keeps the codes. */
int orc_quantize_fp8_pack(const float* in, uint8_t* out, float* scale, size_t rows, size_t cols) {
  if (rows == 0 || cols == 0 || cols % 4 != 0) return -1;
  for (size_t r = 0; r < rows; ++r) {
    const float* x = in + r * cols;
    const float s = row_scale(x, cols);
    scale[r] = s;
    for (size_t c = 0; c < cols; ++c) out[r * cols + c] = orc_fp32_to_fp8e4m3(clamp448(x[c] / s));
  }
  return 0;
}

/* quant.cpp:231-243: bits += 0x7FFF + lsb; mask. */
int orc_round_bf16(float* x, size_t n) {
  if (n == 0) return -1;
  for (size_t i = 0; i < n; ++i) {
    uint32_t u = float_to_bits(x[i]);
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    x[i] = bits_to_float(u);
  }
  return 0;
}

/* RmsNormRef, src/core/numerics/norm.cpp:7-32: squares added in order with fma, the gain
 * 1 / sqrt(mean + eps), y = (x * gain) * w. */
int orc_rmsnorm(const float* x, const float* w, float* y, size_t rows, size_t cols, float eps) {
  if (rows == 0 || cols == 0 || eps < 0.0f) return -2;
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float mean = 0.0f;
    for (size_t c = 0; c < cols; ++c) mean = fmaf(xr[c], xr[c], mean);
    mean /= (float)cols;
    const float gain = 1.0f / sqrtf(mean + eps);
    for (size_t c = 0; c < cols; ++c) y[r * cols + c] = xr[c] * gain * w[c];
  }
  return 0;
}

/* AddRef, src/core/numerics/norm.cpp:196-209 */
int orc_add(const float* a, const float* b, float* o, size_t n) {
  if (n == 0) return -2;
  for (size_t i = 0; i < n; ++i) o[i] = a[i] + b[i];
  return 0;
}

/* SiluMulRef, src/core/numerics/norm.cpp:211-225: silu = g / (1 + exp(-g)) */
int orc_silu_mul(const float* g, const float* u, float* o, size_t n) {
  if (n == 0) return -2;
  for (size_t i = 0; i < n; ++i) {
    const float silu = g[i] / (1.0f + expf(-g[i]));
    o[i] = silu * u[i];
  }
  return 0;
}

/* SigmoidGateRef, src/core/numerics/norm.cpp:96-110 */
int orc_sigmoid_gate(const float* a, const float* g, float* o, size_t n) {
  if (n == 0) return -2;
  for (size_t i = 0; i < n; ++i) o[i] = a[i] / (1.0f + expf(-g[i]));
  return 0;
}

/* L2NormRef, norm.cpp:112-134: squares added in order with fma, gain = scale / sqrt(sum + eps) */
int orc_l2norm(const float* x, float* y, size_t rows, size_t cols, float eps, float scale) {
  if (rows == 0 || cols == 0 || eps < 0.0f) return -2;
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float sum = 0.0f;
    for (size_t c = 0; c < cols; ++c) sum = fmaf(xr[c], xr[c], sum);
    const float gain = scale / sqrtf(sum + eps);
    for (size_t c = 0; c < cols; ++c) y[r * cols + c] = xr[c] * gain;
  }
  return 0;
}

/* RmsNormGatedRef, norm.cpp:136-164 */
int orc_rmsnorm_gated(const float* x, const float* w, const float* gate, float* y, size_t rows, size_t cols, float eps) {
  if (rows == 0 || cols == 0 || eps < 0.0f) return -2;
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    const float* gr = gate + r * cols;
    float mean = 0.0f;
    for (size_t c = 0; c < cols; ++c) mean = fmaf(xr[c], xr[c], mean);
    mean /= (float)cols;
    const float gain = 1.0f / sqrtf(mean + eps);
    for (size_t c = 0; c < cols; ++c) {
      const float silu = gr[c] / (1.0f + expf(-gr[c]));
      y[r * cols + c] = xr[c] * gain * w[c] * silu;
    }
  }
  return 0;
}

/* SsmGateRef, norm.cpp:228-251 */
int orc_ssm_gate(const float* a_log, const float* dt, const float* alpha_raw, const float* beta_raw, float* alpha,
                 float* beta, size_t heads, size_t rows) {
  if (heads == 0 || rows == 0) return -2;
  for (size_t r = 0; r < rows; ++r)
    for (size_t h = 0; h < heads; ++h) {
      const size_t i = r * heads + h;
      const float raw = alpha_raw[i] + dt[h];
      const float softplus = raw > 20.0f ? raw : log1pf(expf(raw));
      alpha[i] = expf(a_log[h] * softplus);
      beta[i] = 1.0f / (1.0f + expf(-beta_raw[i]));
    }
  return 0;
}

/* QGateSplitRef, src/core/numerics/attention.cpp:290-313 */
int orc_qgate_split(const float* fused, float* q, float* gate, size_t heads, size_t head_dim, size_t rows) {
  if (heads == 0 || head_dim == 0 || rows == 0) return -2;
  for (size_t rh = 0; rh < rows * heads; ++rh)
    for (size_t e = 0; e < head_dim; ++e) {
      q[rh * head_dim + e] = fused[rh * 2 * head_dim + e];
      gate[rh * head_dim + e] = fused[rh * 2 * head_dim + head_dim + e];
    }
  return 0;
}

/* RepeatHeadsRef, attention.cpp:315-334 (one row) */
int orc_repeat_heads(const float* in, float* out, size_t num_v_heads, size_t head_k_dim, size_t factor) {
  if (num_v_heads == 0 || head_k_dim == 0 || factor == 0 || num_v_heads % factor != 0) return -2;
  const size_t num_k_heads = num_v_heads / factor;
  for (size_t h = 0; h < num_v_heads; ++h)
    for (size_t e = 0; e < head_k_dim; ++e) out[h * head_k_dim + e] = in[(h % num_k_heads) * head_k_dim + e];
  return 0;
}

/* MropeRef, src/core/numerics/attention.cpp: NeoX pairs (j, j + rope_dim/2); pair j turns by the position of
 * its section times theta^(-2j/rope_dim); angle, cosine and sine in double, products in fp32. */
int orc_mrope(float* io, const uint64_t* pos, size_t rows, size_t heads, size_t head_dim, size_t rope_dim, size_t sec_t,
              size_t sec_h, size_t sec_w, double theta) {
  if (rows == 0 || heads == 0 || head_dim == 0 || rope_dim == 0 || rope_dim > head_dim || (rope_dim % 2) != 0 || !(theta > 0.0))
    return -2;
  const size_t pairs = rope_dim / 2;
  if (sec_t + sec_h + sec_w > pairs) return -2;
  for (size_t r = 0; r < rows; ++r)
    for (size_t h = 0; h < heads; ++h) {
      float* base = io + (r * heads + h) * head_dim;
      for (size_t j = 0; j < pairs; ++j) {
        const uint64_t p = j < sec_t ? pos[r * 3] : j < sec_t + sec_h ? pos[r * 3 + 1] : pos[r * 3 + 2];
        const double angle = (double)p * pow(theta, -2.0 * (double)j / (double)rope_dim);
        const float c = (float)cos(angle), sn = (float)sin(angle);
        const float x1 = base[j], x2 = base[j + pairs];
        base[j] = x1 * c - x2 * sn;
        base[j + pairs] = x1 * sn + x2 * c;
      }
    }
  return 0;
}

/* GemmF32Ref / GemmBf16Ref, src/core/numerics/gemm.cpp:205-252: c[i][j] = fma chain over t of a[i][t] and w[j][t]
 * (bf16 weights widened to fp32) */
int orc_gemm_dense(int bf16, const float* a, const void* w, float* c, size_t m, size_t n, size_t k) {
  if (m == 0 || n == 0 || k == 0) return -2;
#pragma omp parallel for collapse(2) schedule(static)
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (size_t t = 0; t < k; ++t) {
        const float wf = bf16 ? orc_bf16_to_float(((const uint16_t*)w)[j * k + t]) : ((const float*)w)[j * k + t];
        acc = fmaf(a[i * k + t], wf, acc);
      }
      c[i * n + j] = acc;
    }
  return 0;
}

/* RopeRef, src/core/numerics/attention.cpp:11-43: row r at position pos_base + r, NeoX pairs (j, j + rope_dim / 2) */
int orc_rope(float* io, size_t rows, size_t heads, size_t head_dim, size_t rope_dim, uint64_t pos_base, double theta) {
  if (rows == 0 || heads == 0 || head_dim == 0 || rope_dim == 0 || rope_dim > head_dim || (rope_dim % 2) != 0 || !(theta > 0.0))
    return -2;
  const size_t half = rope_dim / 2;
  for (size_t r = 0; r < rows; ++r) {
    const double pos = (double)(pos_base + r);
    for (size_t h = 0; h < heads; ++h) {
      float* base = io + (r * heads + h) * head_dim;
      for (size_t j = 0; j < half; ++j) {
        const double angle = pos * pow(theta, -2.0 * (double)j / (double)rope_dim);
        const float c = (float)cos(angle), sn = (float)sin(angle);
        const float x1 = base[j], x2 = base[j + half];
        base[j] = x1 * c - x2 * sn;
        base[j + half] = x1 * sn + x2 * c;
      }
    }
  }
  return 0;
}

/* QuantizeQ8Ref / QuantizeQ4Ref, src/core/numerics/quant.cpp:123-181: limit 127 (bytes) or 7 (nibbles, element 2i low) */
int orc_quantize_rows(int kind, const float* in, uint8_t* out, float* scale, size_t rows, size_t cols) {
  if (rows == 0 || cols == 0 || (kind != 0 && kind != 1) || cols % (kind == 0 ? 4 : 8) != 0) return -2;
  const long limit = kind == 0 ? 127 : 7;
  for (size_t r = 0; r < rows; ++r) {
    float amax = 0.0f;
    for (size_t c = 0; c < cols; ++c) {
      const float v = fabsf(in[r * cols + c]);
      if (amax < v) amax = v;
    }
    const float s = amax > 0.0f ? amax / (float)limit : 1.0f;
    scale[r] = s;
    for (size_t c = 0; c < cols; ++c) {
      long q = lroundf(in[r * cols + c] / s);
      if (q < -limit) q = -limit;
      if (q > limit) q = limit;
      if (kind == 0) {
        out[r * cols + c] = (uint8_t)(int8_t)q;
      } else {
        uint8_t* b = out + (r * cols + c) / 2;
        const uint8_t nib = (uint8_t)((uint8_t)q & 0xF);
        *b = (c % 2 == 0) ? nib : (uint8_t)(*b | (nib << 4));
      }
    }
  }
  return 0;
}

/* DeltaStepHeadsRef, attention.cpp: per head and state column d: read = sum_j S[j][d] k[j] (fma, in order);
 * S[j][d] <- alpha (S[j][d] - beta k[j] read) + beta v[d] k[j]; o[d] = sum_j S'[j][d] q[j]. */
int orc_delta_step_heads(float* s, const float* k, const float* v, const float* q, float* o, const float* alpha,
                         const float* beta, size_t heads, size_t dk, size_t dv) {
  if (heads == 0 || dk == 0 || dv == 0) return -2;
  for (size_t h = 0; h < heads; ++h) {
    float* st = s + h * dk * dv;
    const float *kh = k + h * dk, *qh = q + h * dk, *vh = v + h * dv;
    for (size_t d = 0; d < dv; ++d) {
      float read = 0.0f;
      for (size_t j = 0; j < dk; ++j) read = fmaf(st[j * dv + d], kh[j], read);
      float out = 0.0f;
      for (size_t j = 0; j < dk; ++j) {
        const float updated = alpha[h] * (st[j * dv + d] - beta[h] * kh[j] * read) + beta[h] * vh[d] * kh[j];
        st[j * dv + d] = updated;
        out = fmaf(updated, qh[j], out);
      }
      o[h * dv + d] = out;
    }
  }
  return 0;
}

/* Element idx of a key / value cache as fp32.  kv_format: 0 fp32, 1 binary16, 2 int8, 3 two's-complement nibble
 * (bits 4 (idx % 2) of byte idx / 2), 4 FP8 E4M3; formats 2..4 times the scale of the element's key row
 * (AttentionRefF16, AttentionQ8Ref, AttentionQ4Ref, AttentionFp8Ref: src/core/numerics/attention.cpp:45-157). */
static float cache_element(int kv_format, const void* cache, size_t idx, float scale) {
  const uint8_t* b = (const uint8_t*)cache;
  switch (kv_format) {
    case 0: return ((const float*)cache)[idx];
    case 1: return orc_fp16_to_float((uint16_t)(b[2 * idx] | ((uint16_t)b[2 * idx + 1] << 8)));
    case 2: return (float)(int8_t)b[idx] * scale;
    case 3: {
      int v = (b[idx / 2] >> ((idx % 2) * 4)) & 0xF;
      if (v & 0x8) v -= 16;
      return (float)v * scale;
    }
    default: return orc_fp8e4m3_to_float(b[idx]) * scale;
  }
}

/* AttentionRef, src/core/numerics/attention.cpp:159-214: per query row i (position q_base + i) and head h: scores
 * fma(q, k) * 1/sqrt(head_dim) over keys start..last, the row's max, exp(score - max), their sum in key order, then
 * out[e] = fma(score / sum, v[e]) in key order.  The cache is decoded first, as the reference's wrappers do. */
int orc_attention(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                  float* out, size_t m, size_t n, size_t heads, size_t kv_heads, size_t head_dim, uint64_t q_base,
                  size_t window, int causal) {
  if (m == 0 || n == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || heads % kv_heads != 0) return -2;
  if (kv_format < 0 || kv_format > 4 || (kv_format >= 2 && (!k_scale || !v_scale))) return -2;
  const size_t row = kv_heads * head_dim, group = heads / kv_heads;
  float* kf = (float*)malloc(n * row * sizeof(float));
  float* vf = (float*)malloc(n * row * sizeof(float));
  float* scores = (float*)malloc(n * sizeof(float));
  if (!kf || !vf || !scores) {
    free(kf), free(vf), free(scores);
    return -1;
  }
  for (size_t j = 0; j < n; ++j)
    for (size_t d = 0; d < row; ++d) {
      kf[j * row + d] = cache_element(kv_format, k, j * row + d, kv_format >= 2 ? k_scale[j] : 1.0f);
      vf[j * row + d] = cache_element(kv_format, v, j * row + d, kv_format >= 2 ? v_scale[j] : 1.0f);
    }
  const float scale = 1.0f / sqrtf((float)head_dim);
  for (size_t i = 0; i < m; ++i) {
    const size_t pos = (size_t)(q_base + i);
    const size_t last = causal ? (pos >= n ? n - 1 : pos) : n - 1;
    size_t start = 0;
    if (causal) {
      start = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
      if (start > last) start = last;
    }
    for (size_t h = 0; h < heads; ++h) {
      const size_t kvh = h / group;
      const float* qr = q + (i * heads + h) * head_dim;
      float top = 0.0f;
      for (size_t j = start; j <= last; ++j) {
        const float* kr = kf + (j * kv_heads + kvh) * head_dim;
        float dot = 0.0f;
        for (size_t e = 0; e < head_dim; ++e) dot = fmaf(qr[e], kr[e], dot);
        dot *= scale;
        scores[j] = dot;
        if (j == start || dot > top) top = dot;
      }
      float denom = 0.0f;
      for (size_t j = start; j <= last; ++j) {
        scores[j] = expf(scores[j] - top);
        denom += scores[j];
      }
      float* o = out + (i * heads + h) * head_dim;
      for (size_t e = 0; e < head_dim; ++e) {
        float acc = 0.0f;
        for (size_t j = start; j <= last; ++j) acc = fmaf(scores[j] / denom, vf[(j * kv_heads + kvh) * head_dim + e], acc);
        o[e] = acc;
      }
    }
  }
  free(kf), free(vf), free(scores);
  return 0;
}

/* Conv1dStepRef, src/core/numerics/conv.cpp: y[c] = sum_i w[c][i] * x[c][i], fma in order (x newest first) */
int orc_conv1d_step(const float* x, const float* w, float* y, size_t channels, size_t width) {
  if (channels == 0 || width == 0) return -2;
  for (size_t c = 0; c < channels; ++c) {
    float acc = 0.0f;
    for (size_t i = 0; i < width; ++i) acc = fmaf(w[c * width + i], x[c * width + i], acc);
    y[c] = acc;
  }
  return 0;
}

/* conv1d_state (device contract, rocm_kernels_basic.cpp:2193-2245): per channel, W in checkpoint tap order
 * (tap 0 oldest), history newest first; acc = w[last] * current, then fma over the history; SiLU; q/k/v split;
 * history shifted; optional copy of row t's history to slot t + 1 of hist_hist. */
int orc_conv1d_state(const float* qkv, const float* w, float* hist, float* q, float* k, float* v, float* hist_hist,
                     size_t conv_dim, size_t width, size_t key_dim, size_t qkv_offset, size_t rows, size_t hist_stride) {
  if (conv_dim == 0 || width == 0 || rows == 0 || 2 * key_dim > conv_dim) return -2;
  const size_t stride = width - 1, value_dim = conv_dim - 2 * key_dim;
  for (size_t c = 0; c < conv_dim; ++c) {
    const size_t hbase = c * stride;
    for (size_t t = 0; t < rows; ++t) {
      const float current = qkv[qkv_offset + t * conv_dim + c];
      float acc = w[c * width + (width - 1)] * current;
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
  return 0;
}

/* top_k_rows (rocm_kernels.hpp:558-566): the top_k largest of each row, descending; equal values: lowest index first */
int orc_top_k_rows(const float* logits, uint32_t* ids, float* vals, size_t rows, size_t vocab, size_t top_k, size_t row_base) {
  if (rows == 0 || vocab == 0 || top_k == 0 || top_k > 32) return -2;
  for (size_t r = 0; r < rows; ++r) {
    const float* row = logits + (row_base + r) * vocab;
    for (size_t p = 0; p < top_k; ++p) {
      size_t arg = (size_t)-1;
      float best = -INFINITY;
      for (size_t c = 0; c < vocab; ++c) {
        int used = 0;
        for (size_t t = 0; t < p; ++t) used |= ids[r * top_k + t] == (uint32_t)c && vals[r * top_k + t] == row[c];
        if (used) continue;
        if (arg == (size_t)-1 || row[c] > best) {
          best = row[c];
          arg = c;
        }
      }
      ids[r * top_k + p] = arg == (size_t)-1 ? 0u : (uint32_t)arg;
      vals[r * top_k + p] = arg == (size_t)-1 ? -INFINITY : best;
    }
  }
  return 0;
}

/* ------------------------------------------------------------ routed experts */

/* moe_gate (rocm_kernels_basic.cpp:1896-1929): softmax over the selected logits and the
 * sigmoid of the shared-expert gate x . w.  The device adds the products as a tree; here in order. */
int orc_moe_gate(const float* vals, const float* x, const float* w, float* wts, float* sig, size_t top_k, size_t hidden) {
  if (top_k == 0 || hidden == 0) return -2;
  float dot = 0.0f;
  for (size_t t = 0; t < hidden; ++t) dot += x[t] * w[t];
  float m = -3.402823466e+38f;
  for (size_t p = 0; p < top_k; ++p) m = fmaxf(m, vals[p]);
  float sum = 0.0f;
  for (size_t p = 0; p < top_k; ++p) sum += expf(vals[p] - m);
  for (size_t p = 0; p < top_k; ++p) wts[p] = expf(vals[p] - m) / sum;
  sig[0] = 1.0f / (1.0f + expf(-dot));
  return 0;
}

/* moe_scale_add (rocm_kernels_basic.cpp:1931-1942): o = a + f[idx] * b */
int orc_moe_scale_add(const float* a, const float* b, const float* f, float* o, size_t n, size_t idx) {
  if (n == 0) return -2;
  for (size_t i = 0; i < n; ++i) o[i] = a[i] + f[idx] * b[i];
  return 0;
}

/* moe_experts_gate_up_q4k (rocm_kernels_moe.cpp:15-46): phi[slot][j] = silu(G_e[j] . x) * (U_e[j] . x),
 * e = ids[slot]; the dots are those of GemmQ4KRef. */
int orc_moe_experts_gate_up_q4k(const float* x, const uint8_t* gate, const uint8_t* up, const uint32_t* ids, float* phi,
                                size_t hidden, size_t inter, size_t top_k, size_t gate_stride, size_t up_stride) {
  if (hidden == 0 || hidden % 256 != 0 || inter == 0 || top_k == 0) return -2;
  float* g = (float*)malloc(2 * inter * sizeof(float));
  if (!g) return -1;
  float* u = g + inter;
  for (size_t slot = 0; slot < top_k; ++slot) {
    const size_t e = ids[slot];
    orc_gemm_q4k(x, gate + e * gate_stride, g, 1, inter, hidden);
    orc_gemm_q4k(x, up + e * up_stride, u, 1, inter, hidden);
    for (size_t j = 0; j < inter; ++j) phi[slot * inter + j] = (g[j] / (1.0f + expf(-g[j]))) * u[j];
  }
  free(g);
  return 0;
}

/* moe_experts_down_q4k / _q6k (rocm_kernels_moe.cpp:48-107): out[j] (+)= sum_slot wts[slot] * (D_e[j] . phi[slot]),
 * slots added in order. */
int orc_moe_experts_down(int fmt, const float* phi, const uint8_t* down, const uint32_t* ids, const float* wts, float* out,
                         size_t hidden, size_t inter, size_t top_k, size_t down_stride, int accumulate) {
  if (hidden == 0 || inter == 0 || inter % 256 != 0 || top_k == 0 || (fmt != 0 && fmt != 1)) return -2;
  float* d = (float*)malloc(2 * hidden * sizeof(float));
  if (!d) return -1;
  float* acc = d + hidden;
  for (size_t j = 0; j < hidden; ++j) acc[j] = 0.0f;
  for (size_t slot = 0; slot < top_k; ++slot) {
    const size_t e = ids[slot];
    if (fmt == 0) orc_gemm_q4k(phi + slot * inter, down + e * down_stride, d, 1, hidden, inter);
    else orc_gemm_q6k(phi + slot * inter, down + e * down_stride, d, 1, hidden, inter);
    for (size_t j = 0; j < hidden; ++j) acc[j] += wts[slot] * d[j];
  }
  for (size_t j = 0; j < hidden; ++j) out[j] = accumulate ? out[j] + acc[j] : acc[j];
  free(d);
  return 0;
}

/* --------------------------------------------------------------- W4A8 fold */

/* E4M3 byte of E2M1 magnitude index i scaled by 2^-d; the table is derived
 * here from its definition and checked against the reference's literal
 * table (quant.cpp:846-863) by the tests: exact value when representable,
 * else rounded to nearest on the subnormal grid of step 2^-9 with ties
 * toward zero (0.5 -> 0, 1.5 -> 1, 0.75 -> 1). */
static uint8_t fold_code(unsigned d, unsigned i) {
  static const unsigned twice[8] = {0, 1, 2, 3, 4, 6, 8, 12}; /* 2 * magnitude */
  if (i == 0) return 0;
  /* value = twice * 2^(-1-d); in units of 2^-9: twice * 2^(8-d) */
  if (d <= 8) {
    unsigned units = twice[i] << (8 - d);
    if (units < 8) return (uint8_t)units; /* subnormal, exact */
    unsigned e = 1;                        /* normal: units = (8+m) * 2^(e-1) */
    while (units >= 16) {
      units >>= 1;
      ++e;
    }
    return (uint8_t)((e << 3) | (units - 8));
  }
  unsigned sh = d - 8;
  return (uint8_t)((twice[i] + (1u << (sh - 1)) - 1u) >> sh); /* ties toward zero */
}

/* mxfp4_row_ref.comp:26-40 / quant.cpp:880-884 */
int orc_mxfp4_row_ref(const uint8_t* scales, uint8_t* wref, size_t rows, size_t cols) {
  if (rows == 0 || cols == 0 || cols % 32 != 0) return -1;
  const size_t nb = cols / 32;
  for (size_t r = 0; r < rows; ++r) {
    uint8_t mx = 0;
    for (size_t b = 0; b < nb; ++b)
      if (scales[r * nb + b] > mx) mx = scales[r * nb + b];
    wref[r] = mx;
  }
  return 0;
}

static uint8_t fold_nibble(uint8_t nib, int ref, int sbyte) {
  int d = ref - sbyte;
  if (d < 0) d = 0;
  if (d > 15) d = 15;
  return (uint8_t)(fold_code((unsigned)d, nib & 7u) | ((nib & 8u) ? 0x80u : 0u));
}

/* quant.cpp:865-899 */
int orc_fold_mxfp4_to_fp8(const uint8_t* w, const uint8_t* scales, uint8_t* out, uint8_t* wref,
                          size_t rows, size_t cols) {
  if (orc_mxfp4_row_ref(scales, wref, rows, cols)) return -1;
  const size_t nb = cols / 32;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      const uint8_t byte = w[(r * cols + c) / 2];
      const uint8_t nib = (c % 2 == 0) ? (byte & 15) : (byte >> 4);
      out[r * cols + c] = fold_nibble(nib, wref[r], scales[r * nb + c / 32]);
    }
  return 0;
}

/* quant.cpp:901-924: C = (sum fp8(a)*fp8(w)) * As[i] * 2^(wref[j]-127). */
int orc_gemm_mxfp4_fp8(const uint8_t* a_fp8, const float* as, const uint8_t* w_fp8,
                       const uint8_t* wref, float* c, size_t m, size_t n, size_t k) {
  if (m == 0 || n == 0 || k == 0) return -1;
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      const float ws = exp2f((float)wref[j] - 127.0f);
      float acc = 0.0f;
      for (size_t t = 0; t < k; ++t)
        acc = fmaf(orc_fp8e4m3_to_float(a_fp8[i * k + t]), orc_fp8e4m3_to_float(w_fp8[j * k + t]),
                   acc);
      c[i * n + j] = acc * as[i] * ws;
    }
  return 0;
}

/* gemm_mxfp4_wmma.comp:78-117: fold inside the kernel from the packed
 * blob||scales buffer; region y covers 128-element chunks
 * [y*per, (y+1)*per), per = ceil(ceil(k/128)/split); plain mul-add. */
int orc_gemm_mxfp4_wmma(const uint8_t* a_fp8, const uint8_t* w_packed, const float* as,
                        const uint8_t* wref, float* c, size_t m, size_t n, size_t k, size_t split) {
  if (m == 0 || n == 0 || k == 0 || k % 32 != 0 || split == 0) return -1;
  const uint8_t* scales = w_packed + n * k / 2;
  const size_t nb = k / 32;
  const size_t chunks = (k + 127) / 128;
  const size_t per = (chunks + split - 1) / split;
  for (size_t y = 0; y < split; ++y) {
    size_t k_lo = y * per * 128;
    size_t k_hi = k_lo + per * 128;
    if (k_hi > k) k_hi = k;
    if (k_lo > k) k_lo = k;
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) {
        float acc = 0.0f;
        for (size_t t = k_lo; t < k_hi; ++t) {
          const uint8_t byte = w_packed[(j * k + t) / 2];
          const uint8_t nib = (t % 2 == 0) ? (byte & 15) : (byte >> 4);
          const uint8_t wb = fold_nibble(nib, wref[j], scales[j * nb + t / 32]);
          acc += orc_fp8e4m3_to_float(a_fp8[i * k + t]) * orc_fp8e4m3_to_float(wb);
        }
        c[y * m * n + i * n + j] = acc * as[i] * ldexpf(1.0f, (int)wref[j] - 127);
      }
  }
  return 0;
}

/* -------------------------------------------------------------- TP reduce */

/* trunk.cpp:226-266: rank 0 adds peer 1, then 2, ... with the add kernel. */
int orc_tp_reduce(const float* const* partials, size_t world, size_t count, float* out) {
  if (world == 0) return -1;
  for (size_t i = 0; i < count; ++i) {
    float acc = partials[0][i];
    for (size_t r = 1; r < world; ++r) acc = acc + partials[r][i];
    out[i] = acc;
  }
  return 0;
}
