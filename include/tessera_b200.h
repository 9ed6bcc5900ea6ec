/*
 * tessera_b200 -- C ABI of the sm_100a CUDA backend for Tessera's quantized
 * projection path.
 *
 * The entry points mirror, one for one, what an implementation of the
 * reference's `tessera::Backend` (include/tessera/backend.hpp:847-1037) has
 * to provide: device set-up, buffers, copies, synchronisation and a
 * name-keyed kernel launch.  The host-side `CudaBackend` class
 * (tessera_b200/backend/cuda_backend.cpp) is a thin C++23 wrapper over these
 * calls; any other host language can bind them directly.
 *
 * Conventions: plain pointers and sizes only; every call returns 0 on
 * success or a positive code equal to the reference's `tessera::StatusCode`
 * (include/tessera/types.hpp:38-48).  All device work of one context is
 * issued on that context's stream, in call order.  Nothing here falls back
 * to the CPU: without a CUDA device every call fails with TSR_DEVICE_ERROR.
 */
#ifndef TESSERA_B200_H_
#define TESSERA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum tsr_status {
  TSR_OK = 0,
  TSR_INVALID_ARGUMENT = 1,
  TSR_UNSUPPORTED_FEATURE = 4,
  TSR_OUT_OF_MEMORY = 5,
  TSR_DEVICE_ERROR = 6
};

/* MemoryKind, include/tessera/backend.hpp:22-25 */
enum tsr_memory_kind { TSR_MEM_DEVICE = 0, TSR_MEM_HOST_VISIBLE = 1 };

typedef struct tsr_context tsr_context;

/* ---- devices: ListGpuNames(), backend.hpp:1066-1071 -------------------- */
int tsr_device_count(int* count);
int tsr_device_name(int device, char* out, size_t capacity);

/* ---- context: Backend::SetDeviceIndex + Init, backend.hpp:871-894 -------
 * tsr_create owns a non-blocking stream.  tsr_create_on_stream borrows a
 * caller-owned cudaStream_t (for hosts that already run a stream). */
int tsr_create(int device_index, tsr_context** out);
int tsr_create_on_stream(int device_index, void* cuda_stream, tsr_context** out);
void tsr_destroy(tsr_context* ctx);
int tsr_context_device(const tsr_context* ctx);
void* tsr_context_stream(const tsr_context* ctx);
/* Backend::DeviceName / MemoryInfo, backend.hpp:853-860 */
int tsr_memory_info(tsr_context* ctx, uint64_t* total_bytes, uint64_t* free_bytes);
/* Text of the last failure on this context (never NULL). */
const char* tsr_last_error(const tsr_context* ctx);

/* ---- buffers: AllocateBuffer / FreeBuffer, backend.hpp:896-912 ----------
 * bytes == 0 is TSR_INVALID_ARGUMENT.  Device allocations are served from a
 * per-context pool so that a mid-step allocation (scratch growth in
 * src/models/qwen3_5/project.cpp:127-138) does not synchronise the device.
 * host_map receives the host address for TSR_MEM_HOST_VISIBLE, else NULL. */
int tsr_alloc(tsr_context* ctx, size_t bytes, int kind, void** handle, void** host_map);
int tsr_free(tsr_context* ctx, int kind, void* handle);

/* ---- copies: CopyH2DAt / CopyD2HAt / CopyD2D / CopyPeerFrom,
 * backend.hpp:918-1003.  h2d returns once `src` is reusable and is ordered
 * before later launches; d2h blocks until the bytes are in `dst`; d2d is
 * stream-ordered and does not block.  Bounds are the caller's (the C++
 * wrapper checks them against Buffer::Size()). */
int tsr_copy_h2d(tsr_context* ctx, void* dst, size_t dst_offset, const void* src, size_t bytes);
int tsr_copy_d2h(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t bytes);
int tsr_copy_d2d(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t dst_offset,
                 size_t bytes);
/* dst lives on ctx's device, src on src_device (peer access is enabled on
 * first use; the copy is complete on return). */
int tsr_copy_peer(tsr_context* ctx, void* dst, int src_device, const void* src, size_t bytes);
/* Backend::Synchronize, backend.hpp:1026 */
int tsr_synchronize(tsr_context* ctx);

/* ---- kernels by name: LoadKernel / LaunchKernel, backend.hpp:1005-1023 --
 * tsr_kernel_lookup returns the id (>= 0) of a built-in or -1 when this
 * backend does not implement the name (the C++ wrapper maps that to
 * UnsupportedFeature, which the reference's callers treat as "fall back",
 * src/core/decode_internal.hpp:1297-1323).
 *
 * tsr_launch binds buffers first, then 64-bit scalars, in the parameter order
 * of the reference's per-kernel contracts (backend.hpp:150-390 and the kernel
 * sources cited beside each id in tessera_b200/csrc/dispatch.cu).  The grid
 * and block of the reference's KernelLaunch are accepted and validated
 * (non-zero) but, like the Vulkan backend with block_*, the launch shape is
 * chosen here from the scalars; only grid_y of the split-K families is
 * meaningful and it must equal the `split` scalar.  buffer_bytes[i] is the
 * size of buffer i; every launch checks it against the bytes the scalars
 * imply and fails with TSR_INVALID_ARGUMENT instead of reading out of range.
 *
 * Ids without a counterpart in the reference's table (this library's own):
 *   gemm_q4k_vec_allreduce, gemm_q6k_vec_allreduce, allreduce_sum: see the
 *     tensor-parallel section below;
 *   gemm_q4k_bf16, gemm_q6k_bf16, gemm_mxfp4_bf16, gemm_fp8_bf16: buffers A (bf16,
 *     m x k), W, [S: fp8 only], C (bf16, m x n); scalars m, n, k (k a multiple of 8).
 *     C = RoundBf16Ref (src/core/numerics/quant.cpp:231-243) of the fp32 id's sums on
 *     the same values; the reference keeps A and C in fp32 (backend.hpp:153-156). */
int tsr_kernel_count(void);
const char* tsr_kernel_name(int kernel);
int tsr_kernel_lookup(const char* name);
int tsr_launch(tsr_context* ctx, int kernel, const uint32_t grid[3], const uint32_t block[3],
               const void* const* buffers, const size_t* buffer_bytes, int n_buffers,
               const uint64_t* scalars, int n_scalars);

/* The same launch as a record, and a call that submits an array of them in order
 * (it stops at the first one that fails and returns that status; *done, when
 * given, receives how many were accepted).  For bindings whose per-call cost is
 * high: a decode loop submits the same few hundred launches every token. */
typedef struct tsr_launch_desc {
  int32_t kernel;
  uint32_t grid[3];
  uint32_t block[3];
  int32_t n_buffers;
  int32_t n_scalars;
  const void* const* buffers;
  const size_t* buffer_bytes;
  const uint64_t* scalars;
} tsr_launch_desc;
int tsr_launch_many(tsr_context* ctx, const tsr_launch_desc* launches, size_t count, size_t* done);

/* ---- deferred submission -------------------------------------------------
 * The reference issues on the order of 500-1000 launches per decoded token
 * (src/backends/rocm/rocm_backend.cpp:697-699) and its Vulkan backend already
 * records launches into a command buffer that is submitted at the next
 * synchronisation point (src/backends/vulkan/vulkan_compute.hpp:117-122).
 * With tsr_set_deferred(ctx, 1), tsr_launch checks its arguments and queues;
 * the queue is issued, in order, by the next copy, tsr_synchronize, tsr_free,
 * tsr_flush or tsr_destroy on the context.  Before it is issued the queue is
 * rewritten where the kernels allow it:
 *   - gemm_q4k_vec / gemm_q6k_vec / gemm_*_rows<R> with a split, followed by the
 *     gemm_vec_reduce of its partial buffer, becomes one launch that writes the
 *     final output (the caller's partial buffer is then not written);
 *   - consecutive Q4_K (or Q6_K) projections that read the same activations with
 *     the same m and k become one launch over up to four weight tensors;
 *   - a silu_mul or rmsnorm whose output is the activation matrix of the Q4_K / Q6_K
 *     projection(s) queued right after it (m <= 8) runs inside that launch's activation
 *     staging; its output buffer is still written;
 *   - an add that follows a single such projection (the _allreduce ids included) and
 *     takes the projection's output as one operand runs in that launch's output stage;
 *     the projection's own output buffer is still written.
 *   A step is only folded when no buffer it writes overlaps one the merged launch
 *   reads (an rmsnorm in place, for instance, stays a launch of its own).
 * A queue that repeats (same kernels, buffers and scalars) is replayed as a CUDA
 * graph from its second appearance on; on = 2 defers and merges without graphs,
 * on = 3 is on = 1 without the folding of silu_mul, rmsnorm and add.
 * Results stay within the projection tolerance of the separate launches but
 * are not bit-identical to them (another split of k).  Hosts that also call
 * the typed launchers below on the same stream must flush first. */
int tsr_set_deferred(tsr_context* ctx, int on);
int tsr_flush(tsr_context* ctx);
/* Counters since the context was created: accepted tsr_launch calls, kernels
 * they became on the device (graph replays included), CUDA graph launches. */
int tsr_launch_stats(tsr_context* ctx, uint64_t* api_launches, uint64_t* device_kernels,
                     uint64_t* graph_launches);
/* One launch for `count` (1..4) projections C_i[m, n_i] = A . dq(W_i)^T that share
 * A (m <= 8 rows of k floats) and the weight format (fmt 0 Q4_K, 1 Q6_K); what
 * the deferred queue emits for QKV or gate/up.  Issued on the context's stream
 * after its queue.  No reference counterpart (one LaunchKernel per projection). */
int tsr_gemv_group(tsr_context* ctx, int fmt, const float* a, const void* const* w, float* const* c,
                   const uint64_t* n, int count, uint64_t m, uint64_t k);

/* ---- typed launchers (what tsr_launch dispatches to) ---------------------
 * `stream` is a cudaStream_t.  Shapes follow C[m,n] = A[m,k] . dq(W[n,k])^T.
 * All pointers are device pointers; A, C and scale vectors need 16-byte
 * alignment, weights 16-byte (Q6_K: 2-byte) alignment. */

/* gemm_q4k_vec, gemm_q4k_rows{2..5}: src/backends/vulkan/kernels/gemm_q4k_vec.comp:66-104,
 * gemm_q4k_rows2.comp:63-109; oracle GemmQ4KRef src/core/numerics/gemm.cpp:62-73.
 * split > 1 writes chunk y of the k range to region y of c (c holds split*m*n floats). */
int tsr_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream);
/* gemm_q6k_vec, gemm_q6k_rows{2..5}: gemm_q6k_vec.comp:49-106; GemmQ6KRef gemm.cpp:88-99 */
int tsr_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream);
/* gemm_vec_reduce: gemm_vec_reduce.comp:20-32 (also gemm_mxfp4_wmma_reduce,
 * src/backends/rocm/rocm_kernels_basic.cpp:1497-1510) */
int tsr_gemm_vec_reduce(const float* part, float* c, uint64_t total, uint64_t split, void* stream);
/* gemm_mxfp4, gemm_mxfp4_rows, gemm_mxfp4_batched: gemm_mxfp4.comp:51-87; GemmMxFp4Ref
 * gemm.cpp:311-344.  w = n*k/2 nibble bytes followed by n*k/32 E8M0 bytes. */
int tsr_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                   void* stream);
/* gemm_fp8: gemm_fp8.comp:52-68; GemmFp8Ref gemm.cpp:253-277 */
int tsr_gemm_fp8(const float* a, const void* w, const float* s, float* c, uint64_t m, uint64_t n,
                 uint64_t k, void* stream);
/* gemm_mxfp4_wmma (W4A8): gemm_mxfp4_wmma.comp:78-117; a = m*k E4M3 bytes, as = m fp32
 * token scales, wref = n E8M0 bytes, c = split regions of m*n. */
int tsr_gemm_mxfp4_w4a8(const void* a_fp8, const void* w, const float* as, const void* wref,
                        float* c, uint64_t m, uint64_t n, uint64_t k, uint64_t split,
                        void* stream);
/* mxfp4_row_ref: mxfp4_row_ref.comp:26-40 */
int tsr_mxfp4_row_ref(const void* w, void* wref, uint64_t n, uint64_t k, void* stream);
/* quantize_fp8: quantize_fp8.comp:74-105; QuantizeFp8Ref src/core/numerics/quant.cpp:180-205 */
int tsr_quantize_fp8(float* data, float* scale, uint64_t rows, uint64_t cols, void* stream);
/* quantize_fp8_pack, quantize_fp8_pack_rows: quantize_fp8_pack_rows.comp:60-95;
 * QuantizeFp8PackRef quant.cpp:207-229 */
int tsr_quantize_fp8_pack(const float* in, void* out, float* scale, uint64_t rows, uint64_t cols,
                          void* stream);
/* round_bf16: round_bf16.comp:14-24; RoundBf16Ref quant.cpp:231-243 */
int tsr_round_bf16(float* x, uint64_t n, void* stream);
/* add, fill: backend.hpp:150-152,258-260 */
int tsr_add(const float* a, const float* b, float* o, uint64_t n, void* stream);
int tsr_fill(int32_t* data, int32_t value, uint64_t n, void* stream);
/* Routed experts of one token (contracts: src/backends/rocm/rocm_kernels.hpp:604-640 of the
 * reference).  ids are read on the device; `experts` bounds them (an id beyond it contributes
 * zero); strides are bytes per expert inside the 3-D expert tensors.
 * moe_gate: wts = softmax(vals[0..top_k)), sig[0] = sigmoid(x . w). */
int tsr_moe_gate(const float* vals, const float* x, const float* w, float* wts, float* sig, uint64_t top_k,
                 uint64_t hidden, void* stream);
/* moe_scale_add: o = a + f[idx] * b */
int tsr_moe_scale_add(const float* a, const float* b, const float* f, float* o, uint64_t n, uint64_t idx,
                      void* stream);
/* moe_experts_gate_up_q4k: phi[slot][j] = silu(G_e[j] . x) * (U_e[j] . x), e = ids[slot] */
int tsr_moe_experts_gate_up_q4k(const float* x, const void* gate, const void* up, const uint32_t* ids, float* phi,
                                uint64_t hidden, uint64_t inter, uint64_t top_k, uint64_t gate_stride,
                                uint64_t up_stride, uint64_t experts, void* stream);
/* moe_experts_down_q4k (fmt 0) / _q6k (fmt 1): out[j] (+)= sum_slot wts[slot] * (D_e[j] . phi[slot]) */
int tsr_moe_experts_down(int fmt, const float* phi, const void* down, const uint32_t* ids, const float* wts,
                         float* out, uint64_t hidden, uint64_t inter, uint64_t top_k, uint64_t down_stride,
                         uint64_t accumulate, uint64_t experts, void* stream);
/* Elementwise / row-wise steps between the projections (contracts: backend.hpp:217-254,386-390;
 * arithmetic: the *Ref functions of src/core/numerics/norm.cpp:96-262, attention.cpp:290-334).
 * sigmoid_gate: O = A * sigmoid(G) */
int tsr_sigmoid_gate(const float* a, const float* g, float* o, uint64_t n, void* stream);
/* l2norm: Y = scale * X / sqrt(sum(X^2) + eps) per row */
int tsr_l2norm(const float* x, float* y, uint64_t rows, uint64_t cols, float eps, float scale, void* stream);
/* rmsnorm_gated: Y[ybase + i] = X[i] / sqrt(mean(X_row^2) + eps) * W[col] * silu(G[gbase + i]) */
int tsr_rmsnorm_gated(const float* x, const float* w, const float* gate, float* y, uint64_t rows, uint64_t cols,
                      float eps, uint64_t gbase, uint64_t ybase, void* stream);
/* ssm_gate: alpha = exp(a_log[h] * softplus(alpha_raw + dt[h])), beta = sigmoid(beta_raw), rows x heads */
int tsr_ssm_gate(const float* a_log, const float* dt, const float* alpha_raw, const float* beta_raw, float* alpha,
                 float* beta, uint64_t heads, uint64_t rows, void* stream);
/* qgate_split: fused rows x heads x (query | gate) -> Q, G */
int tsr_qgate_split(const float* fused, float* q, float* gate, uint64_t heads, uint64_t head_dim, uint64_t rows,
                    void* stream);
/* repeat_heads: out[r][h] = in[r][h % (num_v_heads / factor)] */
int tsr_repeat_heads(const float* in, float* out, uint64_t num_v_heads, uint64_t head_k_dim, uint64_t factor,
                     uint64_t rows, void* stream);
/* embedding_f32 (kind 0) / embedding_bf16 (1) / embedding_q4k (2): out[row] = table[ids[row]] as fp32,
 * a zero row for an id >= vocab; cols a multiple of 256 for Q4_K (backend.hpp:261-265) */
int tsr_embedding(int kind, const uint32_t* ids, const void* table, float* out, uint64_t rows, uint64_t cols,
                  uint64_t vocab, void* stream);
/* mrope: rows x heads x head_dim rotated in place; pos = rows x (t, h, w) u64 (backend.hpp:378-385; MropeRef) */
int tsr_mrope(float* io, const uint64_t* pos, uint64_t rows, uint64_t heads, uint64_t head_dim, uint64_t rope_dim,
              float theta, uint64_t sec_t, uint64_t sec_h, uint64_t sec_w, void* stream);
/* gemm_f32, gemm_f32_batched (bf16 = 0) and gemm_bf16, gemm_bf16_batched, gemm_bf16_wmma, gemm_bf16_rows (bf16 = 1):
 * C (m x n) = A (m x k, fp32) times W^T, W n x k fp32 or bf16, fp32 multiply-adds (backend.hpp:180-190; GemmF32Ref,
 * GemmBf16Ref, src/core/numerics/gemm.cpp:205-252) */
int tsr_gemm_dense(int bf16, const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k, void* stream);
/* rope: rows x heads x head_dim fp32 rotated in place, NeoX pairing over rope_dim, row r at position pos_base + r
 * (backend.hpp:162-166; RopeRef, src/core/numerics/attention.cpp:11-43) */
int tsr_rope(float* io, uint64_t rows, uint64_t heads, uint64_t head_dim, uint64_t rope_dim, uint64_t pos_base, float theta,
             void* stream);
/* quantize_q8 (kind 0) / quantize_q4 (kind 1): per row, scale = amax / 127 (/ 7), codes round-half-away(x / scale)
 * clamped; int8 bytes (cols % 4 == 0), or nibbles with element 2i in the low half of byte i (cols % 8 == 0); the
 * writers of the int8 / 4-bit key-value cache (backend.hpp:283-298; QuantizeQ8Ref, QuantizeQ4Ref,
 * src/core/numerics/quant.cpp:123-181) */
int tsr_quantize_rows(int kind, const float* in, void* out, float* scale, uint64_t rows, uint64_t cols, void* stream);
/* cast_f32_f16: fp32 -> binary16, round to nearest even; n even (backend.hpp:334-336) */
int tsr_cast_f32_f16(const float* in, void* out, uint64_t n, void* stream);
/* delta_step_heads: `rows` gated delta-rule steps on the per-head state (heads x dk x dv at s + sbase, updated
 * in place when sstride = 0, else row t's state goes to sbase + (t+1)*sstride); k, q rows x heads x dk; v, o
 * rows x heads x dv; alpha, beta read at abase + t*heads + h; dk <= 256 (backend.hpp:239-248; DeltaStepHeadsRef) */
int tsr_delta_step_heads(float* s, const float* k, const float* v, const float* q, float* o, const float* alpha,
                         const float* beta, uint64_t heads, uint64_t dk, uint64_t dv, uint64_t rows, uint64_t sbase,
                         uint64_t sstride, uint64_t abase, void* stream);
/* conv1d_state: `rows` steps of the causal depthwise convolution over (width - 1) history samples per channel
 * (newest first, updated in place), SiLU, split into q, k (key_dim each) and v; with hist_stride != 0 row t's
 * history also goes to hist_hist + (t+1)*hist_stride (src/backends/rocm/rocm_kernels_basic.cpp:2193-2245) */
int tsr_conv1d_state(const float* qkv, const float* w, float* hist, float* q, float* k, float* v, float* hist_hist,
                     uint64_t conv_dim, uint64_t width, uint64_t key_dim, uint64_t qkv_offset, uint64_t rows,
                     uint64_t hist_stride, void* stream);
/* top_k_rows: the top_k (<= 32) largest logits of each row, descending, and their indices; output row r reads
 * input row row_base + r; equal values: lowest index first (src/backends/rocm/rocm_kernels.hpp:558-566) */
int tsr_top_k_rows(const float* logits, uint32_t* ids, float* vals, uint64_t rows, uint64_t vocab, uint64_t top_k,
                   uint64_t row_base, void* stream);
/* Key / value cache formats of the attention entry points. */
#define TSR_KV_F32 0  /* fp32 */
#define TSR_KV_F16 1  /* binary16 */
#define TSR_KV_INT8 2 /* int8 bytes, one fp32 scale per key row (k_scale, v_scale) */
#define TSR_KV_INT4 3 /* two's-complement nibbles, element idx in bits 4 (idx % 2) of byte idx / 2, scale per key row */
#define TSR_KV_FP8 4  /* OCP FP8 E4M3 bytes, scale per key row */
/* attention / attention_q8 / attention_q4 / attention_fp8: grouped-query attention of m query rows (row
 * row_base + i of q / out, at position q_base + i) over n key / value rows (n x kv_heads x head_dim); causal: keys
 * max(0, pos + 1 - window)..min(pos, n - 1) (window 0 = all), else all n; scale 1/sqrt(head_dim); head h reads kv head
 * h / (heads / kv_heads); k_scale / v_scale only for the scaled formats.  head_dim 128 or 256 and heads / kv_heads
 * <= 8, else TSR_UNSUPPORTED_FEATURE.  The key range is cut into chunks inside the call (backend.hpp:167-179,283-309;
 * AttentionRef, AttentionRefF16, AttentionQ8Ref, AttentionQ4Ref, AttentionFp8Ref, src/core/numerics/attention.cpp:45-214) */
int tsr_attention(int kv_format, const float* q, const void* k, const void* v, const float* k_scale, const float* v_scale,
                  float* out, uint64_t m, uint64_t n, uint64_t heads, uint64_t kv_heads, uint64_t head_dim, uint64_t q_base,
                  uint64_t row_base, uint64_t window, uint64_t causal, void* stream);
/* attention_split, attention_split_gqa, attention_q8_split / _q4_split / _fp8_split: the first half alone, with the
 * caller's chunk count (<= 64) and partial buffers: chunk s of (row i, head h) at base = (i * heads + h) * split + s
 * writes pacc[base * head_dim ..], pmax[base], psum[base]; an empty chunk writes (0, -1e30, 0)
 * (backend.hpp:309-330; src/backends/rocm/rocm_kernels_basic.cpp:278-330) */
int tsr_attention_split(int kv_format, const float* q, const void* k, const void* v, const float* k_scale,
                        const float* v_scale, float* pacc, float* pmax, float* psum, uint64_t m, uint64_t n, uint64_t heads,
                        uint64_t kv_heads, uint64_t head_dim, uint64_t q_base, uint64_t window, uint64_t causal,
                        uint64_t split, void* stream);
/* attention_combine: out[(i * heads + h) * head_dim + e] = sum_s w_s pacc / sum_s w_s psum, w_s = exp(pmax_s - max pmax)
 * (src/backends/rocm/rocm_kernels_basic.cpp:664-686) */
int tsr_attention_combine(const float* pacc, const float* pmax, const float* psum, float* out, uint64_t m, uint64_t heads,
                          uint64_t head_dim, uint64_t split, void* stream);
/* silu_mul: O = silu(G) * U, backend.hpp:257-260; SiluMulRef src/core/numerics/norm.cpp:211-225 */
int tsr_silu_mul(const float* g, const float* u, float* o, uint64_t n, void* stream);
/* rmsnorm: Y = X / sqrt(mean(X^2) + eps) * W per row, backend.hpp:212-216; RmsNormRef
 * src/core/numerics/norm.cpp:7-32 (eps < 0: TSR_INVALID_ARGUMENT) */
int tsr_rmsnorm(const float* x, const float* w, float* y, uint64_t rows, uint64_t cols, float eps,
                void* stream);
/* Dequantise whole blocks to fp32 with the reference's rounding sequence
 * (bit-exact check of the codecs).  fmt: 0 Q4_K (quant.cpp:656-675), 1 Q6_K
 * (quant.cpp:421-449), 2 MXFP4 packed n x k (quant.cpp:279-297), 3 FP8 E4M3
 * bytes with per-row scale (gemm.cpp:266-270). */
int tsr_dequantize(int fmt, const void* w, const float* row_scale, float* out, uint64_t n,
                   uint64_t k, void* stream);

/* ---- tensor-parallel weight slicing at load time (host memory) ---------------
 * SliceTensor2D / SliceMxFp4, src/core/loaders/tensor_slice.cpp:50-159, for
 * fmt 0 Q4_K, 1 Q6_K, 2 MXFP4 (blob then scales, kept so), 3 FP8 bytes; kind is
 * the reference's ParallelKind (include/tessera/types.hpp:29-34): 0 replicated,
 * 1 column (rows [rows*rank/world, rows*(rank+1)/world)), 2 row (input columns,
 * whole quantisation blocks).  Unlike the reference, a row split need not be
 * even: rank r keeps blocks [nb*r/world, nb*(r+1)/world) of the nb blocks of a
 * row, which equals the reference's range whenever it accepts the split and
 * makes K = 17408 on 8 ranks possible (tensor_slice.cpp:145-147 rejects it).
 * tsr_slice_shape reports the slice's rows, columns, first kept column (the
 * activations of a row-parallel projection are cut with the same range) and
 * byte size; tsr_slice_tensor copies it.  Host pointers; no device is needed. */
int tsr_slice_shape(int fmt, int kind, uint64_t rows, uint64_t cols, int rank, int world,
                    uint64_t* out_rows, uint64_t* out_cols, uint64_t* col_begin, uint64_t* out_bytes);
int tsr_slice_tensor(int fmt, int kind, uint64_t rows, uint64_t cols, int rank, int world,
                     const void* src, size_t src_bytes, void* dst, size_t dst_bytes);
/* The same copy for ranges the caller chose: rows [row_begin, row_end) and columns
 * [col_begin, col_end) (whole blocks).  For shard maps the kind rule cannot express: a
 * row split whose ranks hold multiples of four Q6_K blocks (rows of 210-byte blocks are
 * then 8-byte aligned, which the staged Q6_K kernel needs), or a column split that
 * follows the uneven k ranges of the row-parallel projection it feeds. */
int tsr_slice_range(int fmt, uint64_t rows, uint64_t cols, uint64_t row_begin, uint64_t row_end,
                    uint64_t col_begin, uint64_t col_end, const void* src, size_t src_bytes,
                    void* dst, size_t dst_bytes);

/* ---- split-K Q4_K projection without any device allocation ----------------
 * No counterpart in the reference: there the caller allocates the split-K
 * partial buffer through Backend::AllocateBuffer.
 *
 * For hosts that must not allocate while they run: an engine that has handed
 * out all device memory at load time, or a decode loop that cannot afford
 * the device-wide synchronisation of cudaMalloc.  C[m,n] = A . dq(W)^T is
 * computed as up to eight k chunks whose partial sums live in a fixed 4 MiB
 * array inside the library (every GPU that loads the library holds it until
 * the process exits), followed by the ordered sum of the chunks.  The call
 * makes no cudaMalloc/cudaFree and uses no allocating library routine.
 *   - m*n may not exceed tsr_gemm_q4k_noalloc_max_outputs() (1,048,576);
 *     larger shapes are refused with TSR_INVALID_ARGUMENT.
 *   - The first call on a device looks up the array's device address, and the
 *     first launch of each kernel loads its code: make one call per shape
 *     family at load time, before any stream capture on that device.
 *   - Batches (m >= 9) whose block count k/256 has no divisor up to 8 that
 *     fits the array run unsplit, straight into c, also without allocating.
 *   - All calls on a device share the one array: calls whose kernels can
 *     overlap on the GPU (different streams) race on it.  Nothing needs
 *     clearing between calls; every partial that is read was just written.
 * Same pointer and alignment rules as tsr_gemm_q4k. */
uint64_t tsr_gemm_q4k_noalloc_max_outputs(void);
int tsr_gemm_q4k_noalloc(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                         void* stream);

/* ---- tensor-parallel sum all-reduce over NVLink peer memory ---------------
 * Replaces the rank-0 gather/add/broadcast of TpReduce
 * (src/models/qwen3_5/trunk.cpp:226-266) and the host-staged AllReduceSum
 * (include/tessera/backend.hpp:1048-1058, src/core/buffer.cpp:216-251): every
 * rank pushes its fp32 partial into a slot on every peer, and each rank adds
 * the slots in rank order, so all ranks hold bit-identical sums.
 *
 * One communicator per rank.  tsr_tp_create allocates the rank's exchange
 * memory (cudaMalloc) sized for vectors of up to max_floats.  Ranks living in
 * one process attach each other's block directly (tsr_tp_local_block +
 * tsr_tp_attach_local, peer access is enabled on the way); ranks in separate
 * processes exchange the 64-byte handle of tsr_tp_ipc_handle out of band and
 * call tsr_tp_attach_ipc.  tsr_tp_allreduce sums `count` floats in place
 * (count a multiple of 4, data 16-byte aligned); every rank must issue the
 * same sequence of calls.  It may be captured in a CUDA graph.  Waits on
 * peers are bounded: when one gives up the call still returns and
 * tsr_tp_error_count becomes non-zero.
 *
 * tsr_tp_reduce_allreduce fuses the split-K reduce of a row-parallel projection
 * into the all-reduce: `partials` holds `split` regions of `count` floats (what
 * gemm_*_vec with a split scalar writes); each rank adds its regions in region
 * order (the order of gemm_vec_reduce, decode_internal.hpp:1325-1345) while it
 * pushes, and `out` receives the sum over ranks in rank order: the same bits as
 * gemm_vec_reduce followed by tsr_tp_allreduce, one launch instead of two.  The
 * reference has no such call (it reduces, then TpReduce).
 *
 * max_floats (and world) must be the same on every rank: each rank computes its
 * peers' offsets from its own values, and attaching a peer whose block was made
 * with other values fails with TSR_INVALID_ARGUMENT.
 *
 * tsr_tp_bind makes `comm` the communicator of a context (same device; NULL
 * unbinds).  The kernel ids gemm_q4k_vec_allreduce / gemm_q6k_vec_allreduce
 * (buffers A, W, C; scalars m, n, k) then run a row-parallel projection of this
 * rank's k range and end, in the same launch, with the sum over ranks: the tile
 * that finishes stores its partial sums into every peer, publishes a flag, waits
 * (bounded) for the peers' flags and adds the ranks in rank order.  allreduce_sum
 * (buffer X; scalars m, n) sums an [m][n] matrix in place with the same tiles.
 * Every rank must issue the same sequence of these ids; without a bound
 * communicator they compute the single-rank result. */
typedef struct tsr_tp_comm tsr_tp_comm;
int tsr_tp_bind(tsr_context* ctx, tsr_tp_comm* comm);
int tsr_tp_create(int device, int rank, int world, uint64_t max_floats, tsr_tp_comm** out);
void tsr_tp_destroy(tsr_tp_comm* comm);
int tsr_tp_local_block(tsr_tp_comm* comm, void** block, uint64_t* bytes);
int tsr_tp_ipc_handle(tsr_tp_comm* comm, void* handle64);
int tsr_tp_attach_ipc(tsr_tp_comm* comm, int peer_rank, const void* handle64);
int tsr_tp_attach_local(tsr_tp_comm* comm, int peer_rank, int peer_device, void* peer_block);
int tsr_tp_allreduce(tsr_tp_comm* comm, float* data, uint64_t count, void* stream);
int tsr_tp_reduce_allreduce(tsr_tp_comm* comm, const float* partials, uint64_t split, float* out,
                            uint64_t count, void* stream);
int tsr_tp_error_count(tsr_tp_comm* comm, uint32_t* count);

#ifdef __cplusplus
}
#endif
#endif
