/*
 * CPU oracle for the quantized projection path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels (tests, the smoke check and the
 * benchmark's CPU-baseline leg); nothing in the shipped library links it.
 *
 * Every function restates, in plain C, one function of the reference
 * (Quackster/tessera); the citation beside each declaration is the reference
 * file:line it follows.  Parity is pinned: the restatement is checked against
 * the reference's own compiled host functions (oracle/_ref, built from the
 * reference sources by oracle/Makefile), against the known-answer values in
 * the reference's comments, and against fixtures generated from the
 * reference build (tests/golden).
 */
#ifndef TESSERA_B200_ORACLE_H_
#define TESSERA_B200_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  ORC_Q4K_BLOCK_ELEMS = 256,
  ORC_Q4K_BLOCK_BYTES = 144, /* include/tessera/types.hpp:155 */
  ORC_Q6K_BLOCK_ELEMS = 256,
  ORC_Q6K_BLOCK_BYTES = 210, /* src/core/numerics/gemm.cpp:91-92 */
  ORC_MXFP4_BLOCK = 32
};

/* ---- scalar codecs ---------------------------------------------------- */
float orc_fp16_to_float(uint16_t h);         /* quant.cpp:75-93   */
float orc_bf16_to_float(uint16_t b);         /* quant.cpp:95-100  */
float orc_fp8e4m3_to_float(uint8_t b);       /* quant.cpp:258-277 */
float orc_e8m0_to_float(uint8_t s);          /* quant.cpp:279-281 */
float orc_f4e2m1_to_float(uint8_t nib);      /* quant.cpp:283-297 */
uint8_t orc_fp32_to_fp8e4m3(float v);        /* quant.cpp:299-342 */
uint8_t orc_fp32_to_f4e2m1(float v);         /* quant.cpp:344-386 */
uint16_t orc_fp16_from_float(float v);       /* quant.cpp:102-124 (truncating) */

/* ---- block decoders ---------------------------------------------------- */
void orc_dequant_q4k_block(const uint8_t* block, float* out256); /* quant.cpp:656-675 */
void orc_dequant_q6k_block(const uint8_t* block, float* out256); /* quant.cpp:421-449 */
/* fmt: 0 = Q4_K, 1 = Q6_K.  Decodes nblocks consecutive blocks. */
int orc_dequant_blocks(int fmt, const uint8_t* bytes, size_t nblocks, float* out); /* quant.cpp:808-840 */

/* ---- GEMM references: C[m,n] = A[m,k] . dq(W[n,k])^T, sequential fma ---- */
int orc_gemm_q4k(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k);   /* gemm.cpp:18-41,62-73 */
int orc_gemm_q6k(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k);   /* gemm.cpp:88-99 */
int orc_gemm_mxfp4(const float* a, const uint8_t* w, const uint8_t* s, float* c,
                   size_t m, size_t n, size_t k);                                              /* gemm.cpp:311-344 */
int orc_gemm_fp8(const float* a, const uint8_t* w, const float* s, float* c,
                 size_t m, size_t n, size_t k);                                                /* gemm.cpp:253-277 */
/* Same results as the four above, rows of W spread over OpenMP threads
 * (rows are independent; the k loop order is unchanged). */
int orc_gemm_q4k_mt(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k, int threads);
int orc_gemm_q6k_mt(const float* a, const uint8_t* w, float* c, size_t m, size_t n, size_t k, int threads);
int orc_gemm_mxfp4_mt(const float* a, const uint8_t* w, const uint8_t* s, float* c,
                      size_t m, size_t n, size_t k, int threads);
int orc_gemm_fp8_mt(const float* a, const uint8_t* w, const float* s, float* c,
                    size_t m, size_t n, size_t k, int threads);

/* ---- split-K GEMV contract (device-only behaviour) ---------------------
 * "_vec"/"_rows" kernels with split > 1 write chunk y of the k range to
 * region y of C (offset y*m*n); gemm_vec_reduce sums regions in order.
 * src/backends/vulkan/kernels/gemm_q4k_vec.comp:80-103, gemm_vec_reduce.comp:20-32 */
int orc_gemm_vec_split(int fmt, const float* a, const uint8_t* w, float* part,
                       size_t m, size_t n, size_t k, size_t split);
int orc_gemm_vec_reduce(const float* part, float* c, size_t total, size_t split);
size_t orc_gemm_vec_split_rule(size_t outputs, size_t k, size_t target); /* decode_internal.hpp:866-885 */

/* ---- activation quantisation ------------------------------------------ */
int orc_quantize_fp8(float* data, float* scale, size_t rows, size_t cols);                    /* quant.cpp:180-205 */
int orc_quantize_fp8_pack(const float* in, uint8_t* out, float* scale, size_t rows, size_t cols); /* quant.cpp:207-229 */
int orc_round_bf16(float* x, size_t n);                                                       /* quant.cpp:231-243 */
int orc_rmsnorm(const float* x, const float* w, float* y, size_t rows, size_t cols, float eps);  /* norm.cpp:7-32 */
int orc_add(const float* a, const float* b, float* o, size_t n);                               /* norm.cpp:196-209 */
int orc_silu_mul(const float* g, const float* u, float* o, size_t n);                          /* norm.cpp:211-225 */
int orc_sigmoid_gate(const float* a, const float* g, float* o, size_t n);                      /* norm.cpp:96-110 */
int orc_l2norm(const float* x, float* y, size_t rows, size_t cols, float eps, float scale);    /* norm.cpp:112-134 */
int orc_rmsnorm_gated(const float* x, const float* w, const float* gate, float* y, size_t rows, size_t cols,
                      float eps);                                                              /* norm.cpp:136-164 */
int orc_ssm_gate(const float* a_log, const float* dt, const float* alpha_raw, const float* beta_raw, float* alpha,
                 float* beta, size_t heads, size_t rows);                                      /* norm.cpp:228-251 */
int orc_qgate_split(const float* fused, float* q, float* gate, size_t heads, size_t head_dim, size_t rows); /* attention.cpp:290-313 */
int orc_repeat_heads(const float* in, float* out, size_t num_v_heads, size_t head_k_dim, size_t factor);    /* attention.cpp:315-334 */
int orc_mrope(float* io, const uint64_t* pos, size_t rows, size_t heads, size_t head_dim, size_t rope_dim, size_t sec_t,
              size_t sec_h, size_t sec_w, double theta);                                        /* attention.cpp MropeRef */
/* device-only contracts (src/backends/rocm/rocm_kernels_basic.cpp:2193-2245, 3178-3245) */
int orc_conv1d_state(const float* qkv, const float* w, float* hist, float* q, float* k, float* v, float* hist_hist,
                     size_t conv_dim, size_t width, size_t key_dim, size_t qkv_offset, size_t rows, size_t hist_stride);
int orc_top_k_rows(const float* logits, uint32_t* ids, float* vals, size_t rows, size_t vocab, size_t top_k, size_t row_base);
int orc_conv1d_step(const float* x, const float* w, float* y, size_t channels, size_t width);  /* conv.cpp Conv1dStepRef */
int orc_gemm_dense(int bf16, const float* a, const void* w, float* c, size_t m, size_t n, size_t k); /* gemm.cpp GemmF32Ref (0), GemmBf16Ref (1) */
int orc_rope(float* io, size_t rows, size_t heads, size_t head_dim, size_t rope_dim, uint64_t pos_base, double theta); /* attention.cpp RopeRef */
int orc_quantize_rows(int kind, const float* in, uint8_t* out, float* scale, size_t rows, size_t cols); /* quant.cpp QuantizeQ8Ref (0), QuantizeQ4Ref (1) */
/* attention.cpp AttentionRef and its cache-decoding wrappers; kv_format 0 fp32, 1 fp16, 2 int8, 3 4-bit, 4 FP8 */
int orc_attention(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                  float* out, size_t m, size_t n, size_t heads, size_t kv_heads, size_t head_dim, uint64_t q_base,
                  size_t window, int causal);
/* one gated delta-rule step on every head's state, in place (attention.cpp DeltaStepHeadsRef) */
int orc_delta_step_heads(float* s, const float* k, const float* v, const float* q, float* o, const float* alpha,
                         const float* beta, size_t heads, size_t dk, size_t dv);

/* Routed-expert kernels of one token (contracts only the device backends hold:
 * src/backends/rocm/rocm_kernels.hpp:604-640, rocm_kernels_moe.cpp:15-107,
 * rocm_kernels_basic.cpp:1896-1942).  Strides are bytes per expert. */
int orc_moe_gate(const float* vals, const float* x, const float* w, float* wts, float* sig, size_t top_k, size_t hidden);
int orc_moe_scale_add(const float* a, const float* b, const float* f, float* o, size_t n, size_t idx);
int orc_moe_experts_gate_up_q4k(const float* x, const uint8_t* gate, const uint8_t* up, const uint32_t* ids, float* phi,
                                size_t hidden, size_t inter, size_t top_k, size_t gate_stride, size_t up_stride);
/* fmt: 0 Q4_K, 1 Q6_K */
int orc_moe_experts_down(int fmt, const float* phi, const uint8_t* down, const uint32_t* ids, const float* wts, float* out,
                         size_t hidden, size_t inter, size_t top_k, size_t down_stride, int accumulate);

/* ---- W4A8 fold path ----------------------------------------------------- */
int orc_mxfp4_row_ref(const uint8_t* scales, uint8_t* wref, size_t rows, size_t cols);        /* mxfp4_row_ref.comp:26-40 */
int orc_fold_mxfp4_to_fp8(const uint8_t* w, const uint8_t* scales, uint8_t* out, uint8_t* wref,
                          size_t rows, size_t cols);                                          /* quant.cpp:846-899 */
int orc_gemm_mxfp4_fp8(const uint8_t* a_fp8, const float* as, const uint8_t* w_fp8,
                       const uint8_t* wref, float* c, size_t m, size_t n, size_t k);          /* quant.cpp:901-924 */
/* The device contract: W is the packed blob||scales buffer, folded inside the
 * kernel; split regions of 128-element chunks.  gemm_mxfp4_wmma.comp:78-117 */
int orc_gemm_mxfp4_wmma(const uint8_t* a_fp8, const uint8_t* w_packed, const float* as,
                        const uint8_t* wref, float* c, size_t m, size_t n, size_t k, size_t split);

/* ---- tensor-parallel reduce --------------------------------------------
 * Sum of `world` fp32 vectors in rank order 0,1,2..., as the rank-0
 * gather/add/broadcast does.  src/models/qwen3_5/trunk.cpp:226-266 */
int orc_tp_reduce(const float* const* partials, size_t world, size_t count, float* out);

#ifdef __cplusplus
}
#endif
#endif
