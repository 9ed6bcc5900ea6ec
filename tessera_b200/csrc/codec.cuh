// Device-side codecs of the quantized projection path (sm_100a).
// Each helper states the reference function whose values it reproduces
// (paths are relative to the reference project).
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tsr {

constexpr int kQ4KBlockBytes = 144;  // include/tessera/types.hpp:155
constexpr int kQ6KBlockBytes = 210;  // src/core/numerics/gemm.cpp:92
constexpr int kBlockElems = 256;

// src/core/numerics/quant.cpp:75-93 (binary16 is exact in binary32).
__device__ __forceinline__ float fp16_bits_to_float(uint32_t h) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// src/core/numerics/quant.cpp:258-277.  Every E4M3 value is exact in
// binary16, so the hardware conversion gives the same fp32.
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(__half(h));
}

// src/core/numerics/quant.cpp:279-281: 2^(s-127); s = 0 is the fp32
// subnormal 2^-127 and s = 255 overflows to +inf exactly as ldexp does.
__device__ __forceinline__ float e8m0_to_float(uint32_t s) {
  return __uint_as_float(s == 0 ? 0x00400000u : (s << 23));
}

// src/core/numerics/quant.cpp:283-297.  The three magnitude bits dropped into
// the low exponent/high mantissa bits of a binary16 give mag * 2^-14,
// subnormal case included; the multiply by 2^14 is exact.
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  const unsigned short bits = static_cast<unsigned short>(((nib & 7u) << 9) | ((nib & 8u) << 12));
  return __half2float(__ushort_as_half(bits)) * 16384.0f;
}

// src/core/numerics/quant.cpp:299-342, same arithmetic (frexp, llrint under
// round-to-nearest-even, subnormal mantissa clamped at 7, saturation at 448).
__device__ __forceinline__ uint32_t float_to_e4m3_ref(float v) {
  const uint32_t u = __float_as_uint(v);
  const uint32_t sign = (u >> 31) << 7;
  const uint32_t mag_bits = u & 0x7FFFFFFFu;
  if (mag_bits > 0x7F800000u) return sign | 0x7Fu;
  if (mag_bits == 0) return sign;
  const float mag = __uint_as_float(mag_bits);
  if (mag > 448.0f) return sign | 0x7Fu;
  int ex;
  const float fr = frexpf(mag, &ex);
  int field = ex + 6;
  if (field < 1) {
    long long man = llrintf(mag * 512.0f);
    if (man > 7) man = 7;
    return sign | static_cast<uint32_t>(man);
  }
  long long man = llrintf((fr * 2.0f - 1.0f) * 8.0f);
  if (man == 8) {
    man = 0;
    ++field;
  }
  if (field > 15) field = 15;
  if (field == 15 && man > 6) man = 6;
  return sign | (static_cast<uint32_t>(field) << 3) | static_cast<uint32_t>(man);
}

// Scale/min pair j of a Q4_K block from the 12 packed bytes held as three
// little-endian words (src/core/numerics/quant.cpp:58-70).
__device__ __forceinline__ void q4k_scale_min(const uint32_t s[3], int j, uint32_t& sc,
                                              uint32_t& mn) {
  auto byte = [&](int i) { return (s[i >> 2] >> ((i & 3) * 8)) & 0xFFu; };
  if (j < 4) {
    sc = byte(j) & 63u;
    mn = byte(j + 4) & 63u;
  } else {
    sc = (byte(j + 4) & 15u) | ((byte(j - 4) >> 6) << 4);
    mn = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4);
  }
}

// E4M3 byte of E2M1 magnitude i scaled by 2^-d (the W4A8 fold table,
// src/core/numerics/quant.cpp:846-863): exact when representable, else
// nearest on the 2^-9 subnormal grid with ties toward zero.
__device__ __forceinline__ uint32_t fold_code(uint32_t d, uint32_t i) {
  // 2 * magnitude packed one nibble each: {0,1,2,3,4,6,8,12}
  const uint32_t twice = (0xC8643210u >> (4 * i)) & 15u;
  if (i == 0) return 0;
  if (d <= 8) {
    uint32_t units = twice << (8 - d);
    if (units < 8) return units;
    uint32_t e = 1;
    while (units >= 16) {
      units >>= 1;
      ++e;
    }
    return (e << 3) | (units - 8);
  }
  const uint32_t sh = d - 8;
  return (twice + (1u << (sh - 1)) - 1u) >> sh;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

}  // namespace tsr
