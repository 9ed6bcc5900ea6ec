// C-ABI shim over the reference's own host reference functions
// (tessera::core::*Ref).  TEST INFRASTRUCTURE ONLY.  It is compiled together
// with the reference's src/core/numerics/{quant,gemm,norm}.cpp and
// src/core/loaders/tensor_slice.cpp, taken from where
// the reference checkout lies, into oracle/_ref/libtessera_ref.so by
// oracle/Makefile.  It pins the C restatement in oracle.c and can serve as
// the timed CPU baseline.  No reference source is copied: this file only
// calls the reference's public functions.
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <span>

#include "core/loaders/tensor_slice.hpp"
#include "core/numerics/attention.hpp"
#include "core/numerics/conv.hpp"
#include "core/numerics/gemm.hpp"
#include "core/numerics/moe_cpu.hpp"
#include "core/numerics/norm.hpp"
#include "core/numerics/quant.hpp"

namespace tc = tessera::core;

namespace {
template <typename T>
std::span<const std::byte> Bytes(const T* p, std::size_t n) {
  return {reinterpret_cast<const std::byte*>(p), n};
}
template <typename T>
std::span<std::byte> MutBytes(T* p, std::size_t n) {
  return {reinterpret_cast<std::byte*>(p), n};
}
template <typename E>
int Code(const E& result) {
  return result ? 0 : -static_cast<int>(result.error());
}
}  // namespace

extern "C" {

float ref_fp16_to_float(std::uint16_t h) { return tc::Fp16ToFloat(h); }
float ref_bf16_to_float(std::uint16_t b) { return tc::Bf16ToFloat(b); }
float ref_fp8e4m3_to_float(std::uint8_t b) { return tc::Fp8E4M3ToFloat(b); }
float ref_e8m0_to_float(std::uint8_t s) { return tc::E8M0ToFloat(s); }
float ref_f4e2m1_to_float(std::uint8_t n) { return tc::F4E2M1ToFloat(n); }
std::uint8_t ref_fp32_to_fp8e4m3(float v) { return tc::Fp32ToFp8E4M3Bits(v); }
std::uint8_t ref_fp32_to_f4e2m1(float v) { return tc::Fp32ToF4E2M1Nibble(v); }
std::uint16_t ref_fp16_from_float(float v) { return tc::Fp16FromFloat(v); }

int ref_dequant_blocks(int fmt, const std::uint8_t* bytes, std::size_t nblocks, float* out) {
  const std::size_t bb = fmt == 0 ? 144 : 210;
  for (std::size_t b = 0; b < nblocks; ++b) {
    auto in = Bytes(bytes + b * bb, bb);
    std::span<float> o(out + b * 256, 256);
    if (fmt == 0) {
      tc::DequantizeQ4K(in, o);
    } else if (fmt == 1) {
      tc::DequantizeQ6K(in, o);
    } else {
      return -1;
    }
  }
  return 0;
}

int ref_quantize_q4k(const float* values, std::size_t nblocks, std::uint8_t* out) {
  for (std::size_t b = 0; b < nblocks; ++b) {
    tc::QuantizeQ4K(std::span<const float>(values + b * 256, 256),
                    reinterpret_cast<std::byte*>(out + b * 144));
  }
  return 0;
}

int ref_gemm_q4k(const float* a, const std::uint8_t* w, float* c, std::size_t m, std::size_t n,
                 std::size_t k) {
  return Code(tc::GemmQ4KRef({a, m * k}, Bytes(w, n * (k / 256) * 144), {c, m * n}, m, n, k));
}
int ref_gemm_q6k(const float* a, const std::uint8_t* w, float* c, std::size_t m, std::size_t n,
                 std::size_t k) {
  return Code(tc::GemmQ6KRef({a, m * k}, Bytes(w, n * (k / 256) * 210), {c, m * n}, m, n, k));
}
int ref_gemm_mxfp4(const float* a, const std::uint8_t* w, const std::uint8_t* s, float* c,
                   std::size_t m, std::size_t n, std::size_t k) {
  return Code(tc::GemmMxFp4Ref({a, m * k}, Bytes(w, n * (k / 2)), Bytes(s, n * (k / 32)),
                               {c, m * n}, m, n, k));
}
int ref_gemm_fp8(const float* a, const std::uint8_t* w, const float* s, float* c, std::size_t m,
                 std::size_t n, std::size_t k) {
  return Code(tc::GemmFp8Ref({a, m * k}, Bytes(w, n * k), {s, n}, {c, m * n}, m, n, k));
}
int ref_quantize_fp8(float* data, float* scale, std::size_t rows, std::size_t cols) {
  return Code(tc::QuantizeFp8Ref({data, rows * cols}, {scale, rows}, rows, cols));
}
int ref_quantize_fp8_pack(const float* in, std::uint8_t* out, float* scale, std::size_t rows,
                          std::size_t cols) {
  return Code(tc::QuantizeFp8PackRef({in, rows * cols}, MutBytes(out, rows * cols), {scale, rows},
                                     rows, cols));
}
int ref_round_bf16(float* x, std::size_t n) { return Code(tc::RoundBf16Ref({x, n})); }
int ref_fold_mxfp4_to_fp8(const std::uint8_t* w, const std::uint8_t* scales, std::uint8_t* out,
                          std::uint8_t* wref, std::size_t rows, std::size_t cols) {
  return Code(tc::FoldMxFp4ToFp8(Bytes(w, rows * cols / 2), Bytes(scales, rows * (cols / 32)),
                                 MutBytes(out, rows * cols), MutBytes(wref, rows), rows, cols));
}
int ref_gemm_mxfp4_fp8(const std::uint8_t* a_fp8, const float* as, const std::uint8_t* w_fp8,
                       const std::uint8_t* wref, float* c, std::size_t m, std::size_t n,
                       std::size_t k) {
  return Code(tc::GemmMxFp4Fp8Ref(Bytes(a_fp8, m * k), {as, m}, Bytes(w_fp8, n * k),
                                  Bytes(wref, n), {c, m * n}, m, n, k));
}

int ref_rmsnorm(const float* x, const float* w, float* y, std::size_t rows, std::size_t cols, float eps) {
  return Code(tc::RmsNormRef({x, rows * cols}, {w, cols}, {y, rows * cols}, rows, cols, eps));
}
int ref_add(const float* a, const float* b, float* o, std::size_t n) {
  return Code(tc::AddRef({a, n}, {b, n}, {o, n}, n));
}
int ref_sigmoid_gate(const float* a, const float* g, float* o, std::size_t n) {
  return Code(tc::SigmoidGateRef({a, n}, {g, n}, {o, n}, n));
}
int ref_l2norm(const float* x, float* y, std::size_t rows, std::size_t cols, float eps, float scale) {
  return Code(tc::L2NormRef({x, rows * cols}, {y, rows * cols}, rows, cols, eps, scale));
}
int ref_rmsnorm_gated(const float* x, const float* w, const float* gate, float* y, std::size_t rows, std::size_t cols,
                      float eps) {
  return Code(tc::RmsNormGatedRef({x, rows * cols}, {w, cols}, {gate, rows * cols}, {y, rows * cols}, rows, cols, eps));
}
int ref_ssm_gate(const float* a_log, const float* dt, const float* alpha_raw, const float* beta_raw, float* alpha,
                 float* beta, std::size_t heads, std::size_t rows) {
  return Code(tc::SsmGateRef({a_log, heads}, {dt, heads}, {alpha_raw, rows * heads}, {beta_raw, rows * heads},
                             {alpha, rows * heads}, {beta, rows * heads}, heads, rows));
}
int ref_qgate_split(const float* fused, float* q, float* gate, std::size_t heads, std::size_t head_dim, std::size_t rows) {
  const std::size_t n = rows * heads * head_dim;
  return Code(tc::QGateSplitRef({fused, 2 * n}, {q, n}, {gate, n}, heads, head_dim, rows));
}
int ref_repeat_heads(const float* in, float* out, std::size_t num_v_heads, std::size_t head_k_dim, std::size_t factor) {
  return Code(tc::RepeatHeadsRef({in, (num_v_heads / factor) * head_k_dim}, {out, num_v_heads * head_k_dim}, num_v_heads,
                                 head_k_dim, factor));
}
int ref_mrope(float* io, const std::uint64_t* pos, std::size_t rows, std::size_t heads, std::size_t head_dim,
              std::size_t rope_dim, std::size_t sec_t, std::size_t sec_h, std::size_t sec_w, double theta) {
  return Code(tc::MropeRef({io, rows * heads * head_dim}, {pos, rows * 3}, rows, heads, head_dim, rope_dim, sec_t, sec_h,
                           sec_w, theta));
}
int ref_delta_step_heads(float* s, const float* k, const float* v, const float* q, float* o, const float* alpha,
                         const float* beta, std::size_t heads, std::size_t dk, std::size_t dv) {
  return Code(tc::DeltaStepHeadsRef({s, heads * dk * dv}, {k, heads * dk}, {v, heads * dv}, {q, heads * dk}, {o, heads * dv},
                                    {alpha, heads}, {beta, heads}, heads, dk, dv));
}
int ref_conv1d_step(const float* x, const float* w, float* y, std::size_t channels, std::size_t width) {
  return Code(tc::Conv1dStepRef({x, channels * width}, {w, channels * width}, {y, channels}, channels, width));
}
int ref_gemm_dense(int bf16, const float* a, const void* w, float* c, std::size_t m, std::size_t n, std::size_t k) {
  if (bf16) return Code(tc::GemmBf16Ref({a, m * k}, {static_cast<const std::byte*>(w), n * k * 2}, {c, m * n}, m, n, k));
  return Code(tc::GemmF32Ref({a, m * k}, {static_cast<const float*>(w), n * k}, {c, m * n}, m, n, k));
}
int ref_rope(float* io, std::size_t rows, std::size_t heads, std::size_t head_dim, std::size_t rope_dim, std::uint64_t pos_base,
             double theta) {
  return Code(tc::RopeRef({io, rows * heads * head_dim}, rows, heads, head_dim, rope_dim, pos_base, theta));
}
int ref_quantize_rows(int kind, const float* in, std::uint8_t* out, float* scale, std::size_t rows, std::size_t cols) {
  if (kind == 0) return Code(tc::QuantizeQ8Ref({in, rows * cols}, MutBytes(out, rows * cols), {scale, rows}, rows, cols));
  return Code(tc::QuantizeQ4Ref({in, rows * cols}, MutBytes(out, rows * cols / 2), {scale, rows}, rows, cols));
}
// kv_format as in the C oracle: 0 fp32 (AttentionRef), 1 fp16 (AttentionRefF16), 2 int8 (AttentionQ8Ref),
// 3 4-bit (AttentionQ4Ref), 4 FP8 (AttentionFp8Ref).  Only AttentionRef takes `causal`.
int ref_attention(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                  float* out, std::size_t m, std::size_t n, std::size_t heads, std::size_t kv_heads, std::size_t head_dim,
                  std::uint64_t q_base, std::size_t window, int causal) {
  const std::size_t qn = m * heads * head_dim, count = n * kv_heads * head_dim;
  const auto* kb = static_cast<const std::byte*>(k);
  const auto* vb = static_cast<const std::byte*>(v);
  switch (kv_format) {
    case 0:
      return Code(tc::AttentionRef({q, qn}, {static_cast<const float*>(k), count}, {static_cast<const float*>(v), count},
                                   {out, qn}, m, n, heads, kv_heads, head_dim, q_base, window, causal != 0));
    case 1:
      if (causal == 0) return -2;
      return Code(tc::AttentionRefF16({q, qn}, {kb, count * 2}, {vb, count * 2}, {out, qn}, m, n, heads, kv_heads, head_dim,
                                      q_base, window));
    case 2:
      return Code(tc::AttentionQ8Ref({q, qn}, {kb, count}, {vb, count}, {k_scale, n}, {v_scale, n}, {out, qn}, m, n, heads,
                                     kv_heads, head_dim, q_base, window));
    case 3:
      return Code(tc::AttentionQ4Ref({q, qn}, {kb, count / 2}, {vb, count / 2}, {k_scale, n}, {v_scale, n}, {out, qn}, m, n,
                                     heads, kv_heads, head_dim, q_base, window));
    case 4:
      return Code(tc::AttentionFp8Ref({q, qn}, {kb, count}, {vb, count}, {k_scale, n}, {v_scale, n}, {out, qn}, m, n, heads,
                                      kv_heads, head_dim, q_base, window));
    default: return -2;
  }
}
int ref_silu_mul(const float* g, const float* u, float* o, std::size_t n) {
  return Code(tc::SiluMulRef({g, n}, {u, n}, {o, n}, n));
}

// CpuMoeExpertsForward (src/core/numerics/moe_cpu.cpp:66-131): acc += sum_c wts[c] * expert_c(x).
// gate_dtype / up_dtype / down_dtype are the reference's DType values (Q4K 10, Q6K 12).
int ref_moe_experts_forward(const float* x, const std::uint32_t* experts, const float* wts, std::size_t count,
                            int gate_dtype, const std::uint8_t* gate, std::size_t gate_bytes, std::size_t gate_per,
                            int up_dtype, const std::uint8_t* up, std::size_t up_bytes, std::size_t up_per,
                            int down_dtype, const std::uint8_t* down, std::size_t down_bytes, std::size_t down_per,
                            std::size_t hidden, std::size_t inter, float* acc) {
  return Code(tc::CpuMoeExpertsForward({x, hidden}, {experts, count}, {wts, count}, static_cast<tessera::DType>(gate_dtype),
                                       Bytes(gate, gate_bytes), gate_per, static_cast<tessera::DType>(up_dtype),
                                       Bytes(up, up_bytes), up_per, static_cast<tessera::DType>(down_dtype),
                                       Bytes(down, down_bytes), down_per, hidden, inter, {acc, hidden}));
}

// SliceTensor2D (src/core/loaders/tensor_slice.cpp:105-159).  Returns the slice's byte count, or
// minus the status code; out_rows/out_cols receive the slice's shape.
long long ref_slice_tensor2d(int dtype, std::size_t rows, std::size_t cols, int kind, int rank, int world,
                             const std::uint8_t* src, std::size_t src_bytes, std::uint8_t* dst,
                             std::size_t dst_bytes, std::size_t* out_rows, std::size_t* out_cols) {
  auto sliced = tc::SliceTensor2D(static_cast<tessera::DType>(dtype), rows, cols,
                                  static_cast<tessera::ParallelKind>(kind), rank, world, Bytes(src, src_bytes));
  if (!sliced) return -static_cast<long long>(sliced.error());
  if (sliced->bytes.size() > dst_bytes) return -1;
  std::memcpy(dst, sliced->bytes.data(), sliced->bytes.size());
  *out_rows = sliced->rows;
  *out_cols = sliced->cols;
  return static_cast<long long>(sliced->bytes.size());
}

}  // extern "C"
