// tcgen05 / TMEM tiles for the small-batch projections (m >= 9: the
// speculative-verify and chunked-prefill shapes, ids gemm_*_batched,
// gemm_*_wmma, gemm_mxfp4_rows/_batched, gemm_fp8).
//
// C[m,n] = A[m,k] . dq(W[n,k])^T with the roles swapped for the tensor core:
// the 128 weight rows of a CTA are the M side of tcgen05.mma (kind::f16, fp32
// accumulate in TMEM), the tokens are the N side.  Each fp32 activation is
// split into two fp16 columns (hi = fp16(a), lo = fp16(a - hi)), so the
// activation keeps ~22 bits (Q4_K / Q6_K batches beyond 64 rows: one column,
// twice the tokens per CTA, see token_chunk); weights are dequantised to fp16 exactly as the
// reference's own tensor-core tile does (src/backends/rocm/rocm_kernels_wmma.cpp:
// 54-80 of the reference: weights dequantised to fp16 in shared memory).
//
// Per CTA: four producer warps (thread = weight row; the operand-B pieces are
// shared out among all 128 threads) dequantise a 64-wide k slab, from raw
// bytes loaded four slabs ahead, into the canonical K-major no-swizzle UMMA
// layout (8x16-byte core matrices; leading-byte offset 128 B along k, stride
// byte offset 1024 B along rows), fence it to the async proxy and signal a
// full barrier; one elected thread issues four K=16 MMAs per slab and commits
// them to the slab's empty barrier; two slab buffers overlap dequantisation
// with the MMAs.  The producer warps then read the accumulator with tcgen05.ld
// (warp w owns TMEM lanes 32*(w%4)..), add the hi and lo columns and store C.
// Every wait is bounded and TMEM is always released.
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <cuda_runtime.h>

#include "codec.cuh"
#include "launch.h"
#include "pipeline.cuh"
#include "tessera_b200.h"

namespace tsr {

__device__ unsigned int g_umma_timeouts = 0;

namespace {

constexpr int kTileM = 128;       // weight rows per CTA
constexpr int kSlab = 64;         // k elements per pipeline step
constexpr int kMaxTokens = 64;    // tokens per CTA (N = 2 * padded tokens <= 128)
constexpr int kProducerThreads = 256;  // two per weight row
constexpr int kUmmaThreads = kProducerThreads + 96;  // + the MMA warp, the weight TMA warp, the activation copy warp
constexpr int kBSlabPitch = 512 * kSlab * 2;  // bytes per slab of pre-converted activations: up to 512 operand rows (64 KiB)
constexpr int kASlabBytes = kTileM * kSlab * 2;  // 16384
constexpr int kBufs = 2;                         // slab buffers in shared memory (a power of two)
constexpr int kBufShift = 1;
constexpr uint32_t kLbo = 128, kSbo = (kSlab / 8) * 128;  // bytes

enum Format { kFmtQ4K = 0, kFmtQ6K = 1, kFmtMxFp4 = 2, kFmtFp8 = 3 };

struct UmmaParams {
  const float* a;
  const unsigned char* w;
  const float* scale;  // FP8 row scales
  float* c;
  int m, n, k;
  const unsigned char* bpre;  // activations already in operand layout (convert_activations_kernel), or null
  int split_slabs;            // k is cut among gridDim.z CTAs, this many 64-wide slabs each (a multiple of a ring
                              // stage); CTA z writes its partial sums to region z of c (m x n floats each)
  int one_term;               // batches beyond one chunk: a single binary16 term per activation; 1: 128 tokens per
                              // CTA, 2: 256, 3: 512 as two accumulators of 256 columns (2 and 3 need the
                              // pre-converted activations)
};

// The tokens of chunk `index`: operand-B rows [0, tok_pad) and [tok_pad, 2 tok_pad).  With two terms the first
// half holds the tokens' binary16 values and the second what binary16 lost of them; with one term the rows are
// simply the tokens in order (as the reference's own tensor-core tile has them: binary16 operands,
// src/backends/rocm/rocm_kernels_wmma.cpp:54-80 of the reference).
struct TokenChunk {
  int tok0, tokens, tok_pad;
};
__host__ __device__ __forceinline__ TokenChunk token_chunk(int m, int index, int one_term) {
  const int per = one_term == 3 ? 512 : one_term == 2 ? 256 : one_term == 1 ? 128 : 64;
  TokenChunk c;
  c.tok0 = index * per;
  c.tokens = m - c.tok0 < per ? m - c.tok0 : per;
  c.tok_pad = one_term ? (((c.tokens + 1) / 2 + 7) & ~7) : ((c.tokens + 7) & ~7);
  return c;
}
// Row r of operand B: which token of the chunk, and whether it is the lost-bits row.
__device__ __forceinline__ int row_token(int r, int tok_pad, int one_term, bool* lo_part) {
  *lo_part = !one_term && r >= tok_pad;
  return (one_term || r < tok_pad) ? r : r - tok_pad;
}

// ---- tcgen05 wrappers -------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{.reg .pred p; setp.ne.b32 p, %4, 0; "
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major, no swizzle (layout type 0), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((kLbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((kSbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  return d;
}

// kind::f16: D fp32, A and B fp16, both K-major, M = 128, N = n_cols.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n_cols) {
  return (1u << 4) | ((n_cols >> 3) << 17) | ((kTileM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ---- per-format dequantisation of half a slab (32 consecutive weights) ------
// Two producer threads share a weight row: `half` 0 takes k = 64*slab + 0..31,
// `half` 1 the next 32.  The raw bytes are loaded several slabs ahead
// (RawHalf, registers) so that HBM latency is off the critical path.
// MXFP4 and FP8 convert to binary16 exactly (cvt.rn.f16x2.e2m1x2 / .e4m3x2);
// the MXFP4 block scale is a binary16 multiply (exact: a power of two, within
// the binary16 range for every scale a weight tensor realistically holds; what
// falls outside rounds exactly as the fp32 product rounded to binary16 would);
// the FP8 row scale is applied to the accumulator in the epilogue.  Q4_K:
// nibble -> binary16 by a bit pattern, then one fused multiply-add with the
// sub-block's d*sc and dmin*mn rounded to binary16.  Reference arithmetic:
// src/core/numerics/quant.cpp:656-675, 421-449, 279-297; gemm.cpp:266-270.
struct RawHalf {
  uint4 q[2];
  uint32_t x[4];
};

__device__ __forceinline__ void cvt_e2m1x8_h2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
__device__ __forceinline__ void cvt_e4m3x4_h2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}
__device__ __forceinline__ uint32_t h2_const(float v) {
  const __half2 h = __float2half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int FMT>
__device__ __forceinline__ void load_raw(const UmmaParams& p, int row, int slab, int half, RawHalf& r) {
  if (FMT == kFmtQ4K) {
    const int nb = p.k / 256, b = slab >> 2, g = slab & 3;
    const unsigned char* blk = p.w + (static_cast<size_t>(row) * nb + b) * kQ4KBlockBytes;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    r.x[0] = hdr.x, r.x[1] = hdr.y, r.x[2] = hdr.z, r.x[3] = hdr.w;
    r.q[0] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * g));  // both halves: low / high nibbles
    r.q[1] = __ldg(reinterpret_cast<const uint4*>(blk + 32 + 32 * g));
  } else if (FMT == kFmtMxFp4) {
    const unsigned char* nib = p.w + static_cast<size_t>(row) * (p.k / 2) + slab * 32 + half * 16;
    const unsigned char* scales =
        p.w + static_cast<size_t>(p.n) * (p.k / 2) + static_cast<size_t>(row) * (p.k / 32) + slab * 2 + half;
    r.q[0] = __ldg(reinterpret_cast<const uint4*>(nib));
    r.x[0] = __ldg(scales);
  } else if (FMT == kFmtFp8) {
    const unsigned char* wr = p.w + static_cast<size_t>(row) * p.k + slab * 64 + half * 32;
    r.q[0] = __ldg(reinterpret_cast<const uint4*>(wr));
    r.q[1] = __ldg(reinterpret_cast<const uint4*>(wr + 16));
  }
  // Q6_K: 210-byte blocks are only 2-byte aligned; convert() reads them directly
}

// out: 32 binary16 values as four 16-byte pieces (8 values each), k order.
template <int FMT>
__device__ __forceinline__ void convert(const UmmaParams& p, int row, int slab, int half, const RawHalf& r,
                                        uint4 (&out)[4]) {
  uint32_t h[16];
  if (FMT == kFmtQ4K) {
    const int sb = 2 * (slab & 3) + half;  // sub-block: low nibbles are the even one
    const float d = fp16_bits_to_float(r.x[0] & 0xFFFFu), dmin = fp16_bits_to_float(r.x[0] >> 16);
    const uint32_t s[3] = {r.x[1], r.x[2], r.x[3]};
    uint32_t sc, mn;
    q4k_scale_min(s, sb, sc, mn);
    const uint32_t dl = h2_const(d * static_cast<float>(sc)), ml = h2_const(-dmin * static_cast<float>(mn));
    const uint32_t qw[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t t = (half ? (qw[i] >> 4) : qw[i]) & 0x0F0F0F0Fu;
      // bytes n0..n3 -> binary16 pairs (1024 + n0, 1024 + n1), (1024 + n2, 1024 + n3)
      const uint32_t p01 = __byte_perm(t, 0x64646464u, 0x4140), p23 = __byte_perm(t, 0x64646464u, 0x4342);
      h[2 * i] = hfma2_u32(hsub2_u32(p01, 0x64006400u), dl, ml);
      h[2 * i + 1] = hfma2_u32(hsub2_u32(p23, 0x64006400u), dl, ml);
    }
  } else if (FMT == kFmtQ6K) {
    const int nb = p.k / 256, b = slab >> 2, j = slab & 3, hh = j >> 1, hi = j & 1;
    const unsigned char* blk = p.w + (static_cast<size_t>(row) * nb + b) * kQ6KBlockBytes;
    // the block is 2-byte aligned and every offset below is even: 16-bit loads, two elements each
    const unsigned short* b16 = reinterpret_cast<const unsigned short*>(blk);
    const float d = fp16_bits_to_float(__ldg(b16 + 104));
    const int pp = 2 * hi + half;  // 0..3: which 32-element run of the 128-element half block
    const unsigned short* ql = b16 + 32 * hh + 16 * (pp & 1);
    const unsigned short* qh = b16 + 64 + 16 * hh;
    const uint32_t scw = __ldg(b16 + 96 + 4 * hh + pp);
    const float s0 = d * static_cast<float>(static_cast<signed char>(scw & 0xFFu));
    const float s1 = d * static_cast<float>(static_cast<signed char>(scw >> 8));
#pragma unroll
    for (int l = 0; l < 32; l += 2) {
      const uint32_t lo = __ldg(ql + l / 2), hb = __ldg(qh + l / 2);
      const float sl = l < 16 ? s0 : s1;
      float v[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t byte = (lo >> (8 * e)) & 0xFFu;
        const uint32_t nib = (pp & 2) ? (byte >> 4) : (byte & 15u);
        const int q = static_cast<int>(nib | ((((hb >> (8 * e)) & 0xFFu) >> (2 * pp)) & 3u) << 4) - 32;
        v[e] = sl * static_cast<float>(q);
      }
      h[l / 2] = pack_h2(v[0], v[1]);
    }
  } else if (FMT == kFmtMxFp4) {
    const uint32_t scale = h2_const(e8m0_to_float(r.x[0] & 0xFFu));
    const uint32_t qw[4] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t c[4];
      cvt_e2m1x8_h2(qw[i], c);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[4 * i + e] = hmul2_u32(c[e], scale);
    }
  } else {
    const uint32_t qw[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) cvt_e4m3x4_h2(qw[i], h[2 * i], h[2 * i + 1]);
  }
#pragma unroll
  for (int kc = 0; kc < 4; ++kc) out[kc] = make_uint4(h[4 * kc], h[4 * kc + 1], h[4 * kc + 2], h[4 * kc + 3]);
}

// ---- operand B ------------------------------------------------------------------
// Eight consecutive activations of one token -> one 16-byte piece of binary16:
// the clamped value itself (hi rows) or what binary16 lost of it (lo rows).
__device__ __forceinline__ uint4 convert_b_piece(float4 x0, float4 x1, bool lo_part) {
  const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  float o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float cx = fminf(fmaxf(xs[e], -65504.0f), 65504.0f);
    const float hi = __half2float(__float2half_rn(cx));
    o[e] = lo_part ? fminf(fmaxf(xs[e] - hi, -65504.0f), 65504.0f) : cx;
  }
  return make_uint4(pack_h2(o[0], o[1]), pack_h2(o[2], o[3]), pack_h2(o[4], o[5]), pack_h2(o[6], o[7]));
}

// Converts the activations once per launch into the operand-B layout of every
// (token chunk, slab): out[(chunk * nslabs + slab) * kBSlabPitch + ...], so that the
// tiles fetch a slab with one bulk copy instead of converting it in every CTA.
__global__ void __launch_bounds__(256)
convert_activations_kernel(const float* __restrict__ a, unsigned char* __restrict__ out, int m, int k, int one_term) {
  const int slab = blockIdx.x, chunk = blockIdx.y, nslabs = gridDim.x;
  const TokenChunk tc = token_chunk(m, chunk, one_term);
  const int tok0 = tc.tok0, tokens = tc.tokens, tok_pad = tc.tok_pad, n_cols = 2 * tok_pad;
  unsigned char* dst = out + (static_cast<size_t>(chunk) * nslabs + slab) * kBSlabPitch;
  for (int g = threadIdx.x; g < n_cols * (kSlab / 8); g += blockDim.x) {
    const int r = g >> 3, kc = g & 7;
    bool lo_part;
    const int tok = row_token(r, tok_pad, one_term, &lo_part);
    uint4 piece = make_uint4(0u, 0u, 0u, 0u);
    if (tok < tokens) {
      const float4* src = reinterpret_cast<const float4*>(a + static_cast<size_t>(tok0 + tok) * k + slab * kSlab + kc * 8);
      piece = convert_b_piece(__ldg(src), __ldg(src + 1), lo_part);
    }
    *reinterpret_cast<uint4*>(dst + (r >> 3) * kSbo + (r & 7) * 16 + kc * kLbo) = piece;
  }
}

// ---- raw-weight ring (TMA) ------------------------------------------------------
// With RING the weight bytes of a 128-row tile arrive by tiled TMA copies, a
// stage of several slabs at a time, in a ring of kRawStages stages; the
// producers read their 16-byte pieces from shared memory.  Per-thread global
// loads (thread = row) touch 32 different lines per warp instruction and ran
// at an eighth of the memory rate.  Stage layouts:
//   FP8   [2 segments][128 rows][128 B], 128-byte swizzle       (256 k, 4 slabs)
//   MXFP4 the same for the nibbles (512 k, 8 slabs) + [128 rows][16 scale bytes]
//   Q4_K  [128 rows][144 B]: one block per row                  (256 k, 4 slabs)
// Q6_K (2-byte aligned blocks) and shapes whose k is not a whole number of
// segments keep the direct loads (RING = false).
constexpr int kRawStages = 3;
template <int FMT>
struct RingFmt {
  static constexpr int kSlabsPerStage = FMT == kFmtMxFp4 ? 8 : 4;
  static constexpr int kWeightBytes = FMT == kFmtQ4K ? kTileM * kQ4KBlockBytes : 2 * kTileM * 128;
  static constexpr int kScaleBytes = FMT == kFmtMxFp4 ? kTileM * 16 : 0;
  static constexpr int kStageBytes = kWeightBytes + kScaleBytes;
  static constexpr int kStagePitch = (kStageBytes + 1023) & ~1023;  // stages start on 1 KiB boundaries (swizzle)
};

template <int FMT>
__device__ __forceinline__ void read_raw(const unsigned char* stage, int trow, int si, int half, RawHalf& r) {
  if (FMT == kFmtQ4K) {
    const unsigned char* blk = stage + trow * kQ4KBlockBytes;
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    r.x[0] = hdr.x, r.x[1] = hdr.y, r.x[2] = hdr.z, r.x[3] = hdr.w;
    r.q[0] = *reinterpret_cast<const uint4*>(blk + 16 + 32 * si);
    r.q[1] = *reinterpret_cast<const uint4*>(blk + 32 + 32 * si);
  } else {
    // byte offset of this thread's pieces inside the 256 stage bytes of its row
    const int off = FMT == kFmtFp8 ? si * 64 + half * 32 : si * 32 + half * 16;
    const unsigned char* seg = stage + (off >> 7) * (kTileM * 128) + trow * 128;
    const int c = (off >> 4) & 7, x = trow & 7;
    r.q[0] = *reinterpret_cast<const uint4*>(seg + ((c ^ x) << 4));
    if (FMT == kFmtFp8) r.q[1] = *reinterpret_cast<const uint4*>(seg + (((c + 1) ^ x) << 4));
    if (FMT == kFmtMxFp4) r.x[0] = stage[RingFmt<FMT>::kWeightBytes + trow * 16 + si * 2 + half];
  }
}

template <int FMT, bool RING>
__global__ void __launch_bounds__(kUmmaThreads)
gemm_umma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                 const UmmaParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * kTileM;
  const TokenChunk tc = token_chunk(p.m, blockIdx.y, p.one_term);
  const int tok0 = tc.tok0, tokens = tc.tokens;
  const int tok_pad = tc.tok_pad;             // rows [0, tok_pad) and [tok_pad, 2*tok_pad): see token_chunk
  const int n_cols = 2 * tok_pad;             // multiple of 16, <= 128
  const int b_slab_bytes = n_cols * kSlab * 2;
  constexpr int kRingBytes = RING ? kRawStages * RingFmt<FMT>::kStagePitch : 0;
  unsigned char* const ring = smem;                            // [kRawStages][kStagePitch]
  unsigned char* const a_tiles = smem + kRingBytes;            // [kBufs][kASlabBytes]
  unsigned char* const b_tiles = a_tiles + kBufs * kASlabBytes;  // [kBufs][b_slab_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_tiles + kBufs * b_slab_bytes);
  uint64_t* full = bars;                 // [kBufs] producers -> MMA
  uint64_t* empty = bars + kBufs;        // [kBufs] MMA -> producers
  uint64_t* done = bars + 2 * kBufs;     // accumulator complete
  uint64_t* raw_full = done + 1;         // [kRawStages] TMA -> producers
  uint64_t* raw_empty = raw_full + kRawStages;  // [kRawStages] producers -> TMA
  uint64_t* b_full = raw_empty + kRawStages;    // [kBufs] activation copy -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_full + kBufs);
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(n_cols)) tmem_cols <<= 1;
  const int total_slabs = p.k / kSlab;
  const int s_off = gridDim.z > 1 ? static_cast<int>(blockIdx.z) * p.split_slabs : 0;  // this CTA's first slab
  const int nslabs = gridDim.z > 1 ? min(p.split_slabs, total_slabs - s_off) : total_slabs;
  constexpr int kProducerWarps = kProducerThreads / 32;  // then the MMA warp, the weight TMA warp, the activation copy warp

  if (tid == 0) {
    for (int s = 0; s < kBufs; ++s) {
      mbar_init(&full[s], kProducerThreads / 32);  // one arrival per producer warp
      mbar_init(&empty[s], 1);
      mbar_init(&b_full[s], 1);
    }
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], kProducerThreads / 32);
    }
    mbar_init(done, 1);
    mbar_fence_init();
  }
  if (warp == kProducerWarps) tmem_alloc(tmem_slot, tmem_cols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool failed = false;

  if (warp < kProducerWarps) {
    // ---------------- producers: dequantise A rows, convert B rows ---------
    const int trow = tid & (kTileM - 1), half = tid >> 7;  // warps 0-3: first 32 k of a slab, warps 4-7: the rest
    const int wrow = row0 + trow;
    const bool have_row = wrow < p.n;
    // Without the ring: raw bytes by direct loads, a group of kAhead slabs at a time, one group ahead.
    constexpr int kAhead = 4;
    RawHalf raw[2][kAhead];
    auto load_group = [&](int first_slab, RawHalf (&dst)[kAhead]) {
#pragma unroll
      for (int u = 0; u < kAhead; ++u)
        if (have_row && first_slab + u < nslabs) load_raw<FMT>(p, wrow, s_off + first_slab + u, half, dst[u]);
    };
    if (!RING) {
      load_group(0, raw[0]);
      load_group(kAhead, raw[1]);
    }
    // operand B: the slab has n_cols rows of eight 16-byte pieces; thread t converts pieces
    // t, t + 256, ... (at most kBPieces; eight consecutive threads read 256 consecutive bytes of
    // one token), from activations it loaded two slabs earlier
    const int b_pieces = n_cols * (kSlab / 8);
    constexpr int kBPieces = (2 * kMaxTokens * (kSlab / 8) + kProducerThreads - 1) / kProducerThreads;
    float4 bx[2][kBPieces][2];
    auto load_b = [&](int slab, float4 (&dst)[kBPieces][2]) {
#pragma unroll
      for (int i = 0; i < kBPieces; ++i) {
        const int g = tid + i * kProducerThreads;
        dst[i][0] = dst[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < b_pieces && slab < nslabs) {
          const int r = g >> 3, kc = g & 7;
          bool lo_part;
          const int tok = row_token(r, tok_pad, p.one_term, &lo_part);
          if (tok < tokens) {
            const float4* src =
                reinterpret_cast<const float4*>(p.a + static_cast<size_t>(tok0 + tok) * p.k + (s_off + slab) * kSlab + kc * 8);
            dst[i][0] = __ldg(src);
            dst[i][1] = __ldg(src + 1);
          }
        }
      }
    };
    const bool convert_b = p.bpre == nullptr;
    if (convert_b) {
      load_b(0, bx[0]);
      load_b(1, bx[1]);
    }
    if (RING && !convert_b) {
      // The common case (weights from the ring, activations from the scratch copy) as one
      // rolled loop: nothing here lives in per-slab registers, and the unrolled form
      // below spent a fifth of its issue slots waiting for instruction fetch.
#pragma unroll 1
      for (int s = 0; s < nslabs; ++s) {
        const int buf = s & (kBufs - 1), round = s >> kBufShift;
        if (round > 0 && !mbar_wait(&empty[buf], (round - 1) & 1, &g_umma_timeouts)) {
          failed = true;
          break;
        }
        constexpr int kPer = RingFmt<FMT>::kSlabsPerStage;
        const int st = s / kPer, si = s - st * kPer;
        const int slot = st % kRawStages, rround = st / kRawStages;
        if (si == 0 && !mbar_wait(&raw_full[slot], rround & 1, &g_umma_timeouts)) {
          failed = true;
          break;
        }
        uint4 piece4[4] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u),
                           make_uint4(0u, 0u, 0u, 0u)};
        RawHalf rr;
        read_raw<FMT>(ring + slot * RingFmt<FMT>::kStagePitch, trow, si, half, rr);
        if (have_row) convert<FMT>(p, wrow, s_off + s, half, rr, piece4);
        if (si == kPer - 1 || s == nslabs - 1) {  // this warp is done with the stage
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[slot]);
        }
        unsigned char* a_dst = a_tiles + buf * kASlabBytes + (trow >> 3) * kSbo + (trow & 7) * 16 + half * 4 * kLbo;
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) *reinterpret_cast<uint4*>(a_dst + kc * kLbo) = piece4[kc];
        fence_async_proxy();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[buf]);
      }
    } else
    for (int s0 = 0; s0 < nslabs && !failed; s0 += 2 * kAhead) {
#pragma unroll
      for (int uu = 0; uu < 2 * kAhead; ++uu) {
        const int grp = uu / kAhead, u = uu % kAhead;
        const int s = s0 + uu;
        if (s >= nslabs || failed) break;
        const int buf = s & (kBufs - 1), round = s >> kBufShift;
        if (round > 0 && !mbar_wait(&empty[buf], (round - 1) & 1, &g_umma_timeouts)) {
          failed = true;
          break;
        }
        uint4 piece4[4] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u),
                           make_uint4(0u, 0u, 0u, 0u)};
        if (RING) {
          constexpr int kPer = RingFmt<FMT>::kSlabsPerStage;
          const int st = s / kPer, si = s - st * kPer;
          const int slot = st % kRawStages, rround = st / kRawStages;
          if (si == 0 && !mbar_wait(&raw_full[slot], rround & 1, &g_umma_timeouts)) {
            failed = true;
            break;
          }
          RawHalf rr;
          read_raw<FMT>(ring + slot * RingFmt<FMT>::kStagePitch, trow, si, half, rr);
          if (have_row) convert<FMT>(p, wrow, s_off + s, half, rr, piece4);
          if (si == kPer - 1 || s == nslabs - 1) {  // this warp is done with the stage
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[slot]);
          }
        } else if (have_row) {
          convert<FMT>(p, wrow, s_off + s, half, raw[grp][u], piece4);
          if (u == kAhead - 1) load_group(s + 1 + kAhead, raw[grp]);  // this group's registers are free again
        }
        unsigned char* a_dst = a_tiles + buf * kASlabBytes + (trow >> 3) * kSbo + (trow & 7) * 16 + half * 4 * kLbo;
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) *reinterpret_cast<uint4*>(a_dst + kc * kLbo) = piece4[kc];
        if (convert_b) {
          // operand B from the activations loaded two slabs ago; then reload for slab s + 2
#pragma unroll
          for (int i = 0; i < kBPieces; ++i) {
            const int g = tid + i * kProducerThreads;
            if (g < b_pieces) {
              const int r = g >> 3, kc = g & 7;
              *reinterpret_cast<uint4*>(b_tiles + buf * b_slab_bytes + (r >> 3) * kSbo + (r & 7) * 16 + kc * kLbo) =
                  convert_b_piece(bx[u & 1][i][0], bx[u & 1][i][1], !p.one_term && r >= tok_pad);
            }
          }
          load_b(s + 2, bx[u & 1]);
        }
        // every thread orders its own stores before the async proxy; 256 arrivals on one
        // barrier word would serialise, so one lane per warp arrives for the warp
        fence_async_proxy();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[buf]);
      }
    }
  } else if (warp == kProducerWarps) {
    if (lane == 0) {
      // ---------------- MMA issuer ------------------------------------------
      // at most 256 columns per MMA: a wider chunk runs as two MMAs on the same weight slab, the second
      // into the accumulator columns from 256 on
      const int n_first = n_cols > 256 ? 256 : n_cols, n_second = n_cols - n_first;
      const uint32_t idesc = instr_desc(static_cast<uint32_t>(n_first));
      const uint32_t idesc2 = instr_desc(static_cast<uint32_t>(n_second > 0 ? n_second : 16));
      for (int s = 0; s < nslabs; ++s) {
        const int buf = s & (kBufs - 1), round = s >> kBufShift;
        if (!mbar_wait(&full[buf], round & 1, &g_umma_timeouts) ||
            (p.bpre != nullptr && !mbar_wait(&b_full[buf], round & 1, &g_umma_timeouts))) {
          failed = true;
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(a_tiles + buf * kASlabBytes), b_addr = smem_u32(b_tiles + buf * b_slab_bytes);
#pragma unroll
        for (int kk = 0; kk < kSlab / 16; ++kk) {
          umma_f16(tmem_base, smem_desc(a_addr + kk * 2 * kLbo), smem_desc(b_addr + kk * 2 * kLbo), idesc,
                   (s > 0 || kk > 0) ? 1u : 0u);
          if (n_second > 0)
            umma_f16(tmem_base + 256, smem_desc(a_addr + kk * 2 * kLbo), smem_desc(b_addr + (256 / 8) * kSbo + kk * 2 * kLbo),
                     idesc2, (s > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[buf]);  // the slab buffer is free once these MMAs have read it
      }
      umma_commit(done);
    }
  } else if (warp == kProducerWarps + 1 && RING && lane == 0) {
    // ---------------- TMA issuer: raw weight stages -------------------------
    constexpr int kPer = RingFmt<FMT>::kSlabsPerStage;
    const int nstages = (nslabs + kPer - 1) / kPer;
    for (int st = 0; st < nstages; ++st) {
      const int slot = st % kRawStages, rround = st / kRawStages;
      if (rround > 0 && !mbar_wait(&raw_empty[slot], (rround - 1) & 1, &g_umma_timeouts)) break;
      unsigned char* dst = ring + slot * RingFmt<FMT>::kStagePitch;
      mbar_expect_tx(&raw_full[slot], RingFmt<FMT>::kStageBytes);
      const int sta = s_off / kPer + st;  // the stage's index in the whole k
      if (FMT == kFmtQ4K) {
        tma_load_3d(dst, &wmap, 0, sta, row0, &raw_full[slot]);      // (18 x u64, block, rows)
      } else {
        tma_load_3d(dst, &wmap, 0, row0, 2 * sta, &raw_full[slot]);  // (128 B, rows, segments)
        if (FMT == kFmtMxFp4) tma_load_2d(dst + RingFmt<FMT>::kWeightBytes, &smap, 16 * sta, row0, &raw_full[slot]);
      }
    }
  }

  if (warp == kProducerWarps + 2 && lane == 0 && p.bpre != nullptr) {
    // ---------------- activation copy: one bulk copy per slab ----------------
    const unsigned char* src = p.bpre + (static_cast<size_t>(blockIdx.y) * total_slabs + s_off) * kBSlabPitch;
    for (int s = 0; s < nslabs; ++s) {
      const int buf = s & (kBufs - 1), round = s >> kBufShift;
      if (round > 0 && !mbar_wait(&empty[buf], (round - 1) & 1, &g_umma_timeouts)) break;
      mbar_expect_tx(&b_full[buf], static_cast<uint32_t>(b_slab_bytes));
      bulk_load(b_tiles + buf * b_slab_bytes, src + static_cast<size_t>(s) * kBSlabPitch,
                static_cast<uint32_t>(b_slab_bytes), &b_full[buf]);
    }
  }

  // ---------------- epilogue: TMEM -> registers -> C ------------------------
  if (warp < 4) {
    // warp-uniform, so the aligned TMEM loads below are never reached by part of a warp
    const bool ok = __all_sync(0xFFFFFFFFu, !failed && mbar_wait(done, 0, &g_umma_timeouts));
    tcgen05_fence_after();
    if (ok) {
      const int out_row = row0 + tid;
      float* const cz = p.c + (gridDim.z > 1 ? static_cast<size_t>(blockIdx.z) * p.m * p.n : 0);  // this k range's region
      const float out_scale = (FMT == kFmtFp8 && out_row < p.n) ? __ldg(p.scale + out_row) : 1.0f;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      if (p.one_term) {  // column c is token c of the chunk
        for (int c0 = 0; c0 < n_cols; c0 += 8) {
          float v[8];
          tmem_ld8(lane_addr + c0, v);
          if (out_row < p.n) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c0 + j < tokens) cz[static_cast<size_t>(tok0 + c0 + j) * p.n + out_row] = v[j] * out_scale;
          }
        }
      } else {
        for (int c0 = 0; c0 < tok_pad; c0 += 8) {
          float hi[8], lo[8];
          tmem_ld8(lane_addr + c0, hi);
          tmem_ld8(lane_addr + tok_pad + c0, lo);
          if (out_row < p.n) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c0 + j < tokens) cz[static_cast<size_t>(tok0 + c0 + j) * p.n + out_row] = (hi[j] + lo[j]) * out_scale;
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kProducerWarps) tmem_dealloc(tmem_base, tmem_cols);
}

// ---- tensor maps of the raw ring (cached per weight tensor) ---------------------
struct RingMaps {
  CUtensorMap weights, scales;
};
struct RingKey {
  const void* base;
  uint64_t n, k;
  int fmt;
  bool operator==(const RingKey& o) const { return base == o.base && n == o.n && k == o.k && fmt == o.fmt; }
};
struct RingKeyHash {
  size_t operator()(const RingKey& x) const {
    return std::hash<const void*>()(x.base) ^ (x.n * 0x9E3779B97F4A7C15ull) ^ (x.k << 40) ^ (static_cast<size_t>(x.fmt) << 60);
  }
};
std::mutex g_ring_mutex;
std::unordered_map<RingKey, RingMaps, RingKeyHash> g_ring_maps;

int ring_maps(int fmt, const void* w, uint64_t n, uint64_t k, RingMaps* out) {
  std::lock_guard<std::mutex> lock(g_ring_mutex);
  const RingKey key{w, n, k, fmt};
  auto it = g_ring_maps.find(key);
  if (it != g_ring_maps.end()) {
    *out = it->second;
    return kOk;
  }
  RingMaps maps{};
  int rc;
  if (fmt == kFmtQ4K) {
    const uint64_t nb = k / 256;
    const uint64_t dims[3] = {18, nb, n};
    const uint64_t strides[2] = {kQ4KBlockBytes, nb * kQ4KBlockBytes};
    const uint32_t box[3] = {18, 1, kTileM};
    rc = encode_tensor_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, w, dims, strides, box);
    maps.scales = maps.weights;
  } else {
    const uint64_t row_bytes = fmt == kFmtMxFp4 ? k / 2 : k;
    const uint64_t dims[3] = {128, n, row_bytes / 128};
    const uint64_t strides[2] = {row_bytes, 128};
    const uint32_t box[3] = {128, kTileM, 2};
    rc = encode_tensor_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w, dims, strides, box, true);
    maps.scales = maps.weights;
    if (rc == kOk && fmt == kFmtMxFp4) {
      const uint64_t sdims[2] = {k / 32, n};
      const uint64_t sstrides[1] = {k / 32};
      const uint32_t sbox[2] = {16, kTileM};
      rc = encode_tensor_map(&maps.scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                             static_cast<const unsigned char*>(w) + n * (k / 2), sdims, sstrides, sbox);
    }
  }
  if (rc != kOk) return rc;
  if (g_ring_maps.size() > 65536) g_ring_maps.clear();
  g_ring_maps.emplace(key, maps);
  *out = maps;
  return kOk;
}

// Device scratch for the pre-converted activations, one buffer per (device, stream),
// grown on demand and never freed before exit (a captured graph may hold the pointer).
// Returns null when the stream is being captured and no large enough buffer exists yet:
// the tiles then convert the activations themselves.  The memory comes from the
// stream-ordered pool, so growing it never synchronises the device.
unsigned char* activation_scratch(cudaStream_t st, size_t bytes) { return stream_scratch(st, bytes); }

}  // namespace

// `slot` separates users whose buffers are alive at the same time (0: the tile kernels'
// operands and partial sums; 1: the fp32 copies around a bf16 projection; 2: attention's chunk partials; 3: the
// binary16 tile's partial regions when it cuts k).
unsigned char* stream_scratch(cudaStream_t st, size_t bytes, int slot) {
  struct Entry {
    int device;
    int slot;
    cudaStream_t stream;
    unsigned char* ptr;
    size_t bytes;
  };
  static std::mutex mutex;
  static std::vector<Entry> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mutex);
  for (const Entry& e : table)
    if (e.device == dev && e.slot == slot && e.stream == st && e.bytes >= bytes) return e.ptr;
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &status) != cudaSuccess || status != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return nullptr;
  }
  size_t want = 4u << 20;
  while (want < bytes) want <<= 1;
  void* ptr = nullptr;
  if (cudaMallocAsync(&ptr, want, st) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  table.push_back(Entry{dev, slot, st, static_cast<unsigned char*>(ptr), want});
  return static_cast<unsigned char*>(ptr);
}

namespace {

template <int FMT, bool RING>
int launch_umma_impl(UmmaParams p, const RingMaps& maps, cudaStream_t st, bool allow_scratch) {
  // One binary16 term per activation for batches larger than one two-term chunk where the weights are
  // rounded to binary16 anyway (Q4_K, Q6_K: the error class of the result does not change).  MXFP4 and FP8
  // weights are exact in binary16, so up to 128 rows (verify batches) they keep the second term and with it
  // fp32-like results; prefill-sized batches take one term as well (the reference quantises those
  // activations to FP8 or binary16 itself, src/models/qwen3_5/project.cpp:55-85,307-335 of the reference).
  // Beyond 128 rows a CTA takes 256 tokens, beyond 256 rows 512 where shared memory allows (every dequantised
  // weight slab then feeds 256 or 512 accumulator columns), which needs the activations converted ahead of the tiles.
  const int two_term_rows = (FMT == kFmtQ4K || FMT == kFmtQ6K) ? kMaxTokens : 2 * kMaxTokens;
  const bool narrow = p.m > two_term_rows && std::getenv("TSR_TILE_TWO_TERMS") == nullptr;
  // Tokens per CTA: the widest stage is the cheapest per token, but only while the grid still covers the SMs:
  // relative time of one CTA per stage (measured on Q4_K 17408 x 5120: 491 / 787 / 1018 TFLOP/s at 128 / 256 /
  // 512 tokens per CTA) times the waves its grid needs.  5120 weight rows are 40 row tiles: 512 tokens in
  // one chunk would leave 108 SMs idle, two chunks of 256 finish in two thirds of the time.
  // ... and where the grid of the widest stage still leaves half of the SMs idle (5120 weight rows: 40 row
  // tiles), k is cut among up to four CTAs per tile, whose partial sums gemm_vec_reduce adds.
  int widest = !narrow ? 0 : (p.m > 2 * kMaxTokens && allow_scratch && std::getenv("TSR_TILE_128") == nullptr)
                                 ? ((p.m > 4 * kMaxTokens && std::getenv("TSR_TILE_256") == nullptr) ? 3 : 2) : 1;
  constexpr int kPerStage = RING ? RingFmt<FMT>::kSlabsPerStage : 4;
  const int stages_total = (p.k / kSlab + kPerStage - 1) / kPerStage;
  int ksplit = 1;
  if (std::getenv("TSR_TILE_WIDEST") == nullptr) {  // narrower stages only compete from 256 tokens on; the k cut always
    static const int sms = [] {
      int dev = 0, v = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
      return v > 0 ? v : 148;
    }();
    const double unit[4] = {0.5, 0.509, 0.635, 0.982};
    const long tiles = (p.n + kTileM - 1) / kTileM;
    const int max_split = (allow_scratch && std::getenv("TSR_TILE_NO_KSPLIT") == nullptr) ? 4 : 1;
    double best = 0.0;
    int pick = widest;
    for (int mode = widest; mode >= (widest >= 2 ? 1 : widest); --mode) {
      const long per = static_cast<long>(kMaxTokens) << mode;
      const long ctas = tiles * ((p.m + per - 1) / per);
      for (int sp = 1; sp <= max_split; ++sp) {
        if (sp > 1 && (ctas * sp > sms || stages_total / sp < 16)) break;  // one wave, and enough k left per CTA (4096)
        // a split costs the fill and drain of every CTA's pipeline again and the sum of the partial regions
        const double cost = static_cast<double>((ctas * sp + sms - 1) / sms) * (unit[mode] / sp + (sp > 1 ? 0.06 : 0.0));
        if ((mode == widest && sp == 1) || cost < best * 0.9) best = cost, pick = mode, ksplit = sp;  // must win clearly
      }
    }
    widest = pick;
  }
  p.one_term = widest;
  const int nslabs = p.k / kSlab;
  const size_t ring = RING ? static_cast<size_t>(kRawStages) * RingFmt<FMT>::kStagePitch : 0;
  dim3 grid;
  size_t smem = 0;
  for (;;) {
    const int tok_pad = token_chunk(p.m, 0, p.one_term).tok_pad;  // the first chunk is the largest
    const int per_cta = kMaxTokens << p.one_term;
    smem = 1024 + ring + kBufs * kASlabBytes + kBufs * static_cast<size_t>(2 * tok_pad) * kSlab * 2 + 256;
    grid = dim3(static_cast<unsigned>((p.n + kTileM - 1) / kTileM), static_cast<unsigned>((p.m + per_cta - 1) / per_cta));
    // activations -> operand layout once per launch, when scratch is to be had
    p.bpre = allow_scratch ? activation_scratch(st, static_cast<size_t>(grid.y) * nslabs * kBSlabPitch) : nullptr;
    if (p.one_term >= 2 && (p.bpre == nullptr || smem > 227 * 1024)) {  // no scratch, or the ring leaves no room
      --p.one_term;
      continue;
    }
    break;
  }
  if (int rc = allow_dynamic_smem(reinterpret_cast<const void*>(&gemm_umma_kernel<FMT, RING>), 227 * 1024)) return rc;
  if (p.bpre != nullptr) {
    convert_activations_kernel<<<dim3(nslabs, grid.y), 256, 0, st>>>(p.a, const_cast<unsigned char*>(p.bpre), p.m, p.k, p.one_term);
    if (int rc = check_launch()) return rc;
  }
  float* const out = p.c;
  if (ksplit > 1) {
    // region z of the partial buffer takes k range z; the buffer is another slot of the stream's scratch
    p.split_slabs = (stages_total + ksplit - 1) / ksplit * kPerStage;
    ksplit = (nslabs + p.split_slabs - 1) / p.split_slabs;
    float* part = ksplit > 1 ? reinterpret_cast<float*>(stream_scratch(st, static_cast<size_t>(ksplit) * p.m * p.n * 4, 3)) : nullptr;
    if (part == nullptr) ksplit = 1;
    else p.c = part, grid.z = static_cast<unsigned>(ksplit);
  }
  gemm_umma_kernel<FMT, RING><<<grid, kUmmaThreads, smem, st>>>(maps.weights, maps.scales, p);
  if (int rc = check_launch()) return rc;
  if (ksplit > 1) return tsr_gemm_vec_reduce(p.c, out, static_cast<uint64_t>(p.m) * p.n, static_cast<uint64_t>(ksplit), st);
  return kOk;
}

template <int FMT>
int launch_umma(const UmmaParams& p, cudaStream_t st, bool allow_scratch) {
  // the ring wants whole segments (and 16-byte scale rows for MXFP4) and 16-byte aligned weights
  const bool aligned = (reinterpret_cast<uintptr_t>(p.w) & 15u) == 0;
  const bool ring = aligned && (FMT == kFmtQ4K || (FMT == kFmtFp8 && p.k % 128 == 0) ||
                                (FMT == kFmtMxFp4 && p.k % 512 == 0));
  RingMaps maps{};
  if (ring && FMT != kFmtQ6K) {
    if (int rc = ring_maps(FMT, p.w, static_cast<uint64_t>(p.n), static_cast<uint64_t>(p.k), &maps)) return rc;
    return launch_umma_impl<FMT, FMT != kFmtQ6K>(p, maps, st, allow_scratch);
  }
  return launch_umma_impl<FMT, false>(p, maps, st, allow_scratch);
}

}  // namespace

// fmt: 0 Q4_K, 1 Q6_K, 2 MXFP4 (packed blob||scales), 3 FP8 (+ row scales).
// Returns kUnsupportedFeature when the shape is outside the tile's range.
// With allow_scratch false the launch never asks for device memory: the tiles
// convert the activations themselves instead of reading a pre-converted copy.
int umma_gemm(int fmt, const float* a, const void* w, const float* scale, float* c, uint64_t m, uint64_t n,
              uint64_t k, cudaStream_t st, bool allow_scratch) {
  if (k % kSlab != 0 || (fmt <= 1 && k % 256 != 0)) return kUnsupportedFeature;
  const UmmaParams p{a, static_cast<const unsigned char*>(w), scale, c, static_cast<int>(m),
                     static_cast<int>(n), static_cast<int>(k), nullptr};
  switch (fmt) {
    case kFmtQ4K: return launch_umma<kFmtQ4K>(p, st, allow_scratch);
    case kFmtQ6K: return launch_umma<kFmtQ6K>(p, st, allow_scratch);
    case kFmtMxFp4: return launch_umma<kFmtMxFp4>(p, st, allow_scratch);
    case kFmtFp8: return launch_umma<kFmtFp8>(p, st, allow_scratch);
    default: return kInvalidArgument;
  }
}

int umma_set_error_word(unsigned int* word) { return set_host_error_word(word); }

int umma_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_umma_timeouts, sizeof(unsigned int)) == cudaSuccess ? kOk : kDeviceError;
}

}  // namespace tsr
