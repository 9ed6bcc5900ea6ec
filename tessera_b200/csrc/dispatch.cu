// Typed projection launchers and the name-keyed kernel table.
//
// Every id below is a built-in name of the reference's kernel contract; the
// comment beside it names the reference source that defines the contract.
// One CUDA launcher can serve several ids because the contract is the result
// for the given (buffers, scalars), not the reference's thread mapping.
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "context.h"
#include "launch.h"
#include "tessera_b200.h"

using namespace tsr;

namespace {

bool fits_int(uint64_t v) { return v > 0 && v <= 0x7FFFFFFFull; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Batches of 9..16 activation rows go through the staged GEMV eight rows at a
// time (the weights stream once per eight rows) unless the weight has enough
// rows to give most SMs a 128-row tcgen05 tile (measured at m = 16: 17408 rows
// 42-45 us on the tile against 55-64 us in two staged passes; 5120 rows 40 us
// against 30 us); above 16 rows the tile always amortises its dequantisation better.  `launch(i0, rows)` runs rows
// [i0, i0 + rows) and returns a status.
constexpr uint64_t kStagedRows = 8;
constexpr uint64_t kQ6KStagedRows = 32;  // Q6_K batches up to here run as staged passes of eight rows
uint64_t staged_batch_max() {
  static const uint64_t v = [] {
    const char* e = std::getenv("TSR_STAGED_BATCH_MAX");  // experiments: where the tcgen05 tile takes over
    return e ? static_cast<uint64_t>(std::atoi(e)) : 16u;
  }();
  return v;
}
bool tile_fills_device(uint64_t n) {
  static const int sms = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return ((n + 127) / 128) * 10 >= static_cast<uint64_t>(sms) * 7;
}
// `always_up_to`: batches of at most this many rows take the staged kernel even when the tile would fill the
// device (Q6_K: the tile's producers read the 210-byte blocks with narrow loads and need 160 us for
// 17408 x 5120 whatever m is, a staged pass 20-25 us per eight rows).
template <typename Launch>
int staged_in_chunks(uint64_t m, uint64_t n, Launch launch, uint64_t always_up_to = 0) {
  if (m > always_up_to && (m > staged_batch_max() || tile_fills_device(n))) return kUnsupportedFeature;
  // eight rows per pass; up to eight rows as two passes of four where eight rows of a long k do not fit the
  // kernel's shared memory (k = 17408: the digits of eight activation rows alone are 296 KB)
  for (uint64_t per : {kStagedRows, kStagedRows / 2}) {
    if (per < kStagedRows && m > kStagedRows) break;  // larger batches: the tile (it cuts k among its CTAs)
    int rc = kOk;
    for (uint64_t i0 = 0; i0 < m && rc == kOk; i0 += per) rc = launch(i0, m - i0 < per ? m - i0 : per);
    if (rc != kUnsupportedFeature) return rc;  // kUnsupportedFeature can only come from the first pass
  }
  return kUnsupportedFeature;
}

// One pass of up to eight rows over a k too long for the staged kernel's shared memory in one piece: k is cut
// into `parts` equal block ranges, each range's sums go to a region of a scratch buffer (the kernel's caller
// split, as gemm_*_vec with a split writes them) and gemm_vec_reduce adds the regions.
template <typename Staged>
int staged_pass_cut(uint64_t rows, uint64_t n, uint64_t k, float* c, cudaStream_t st, Staged staged) {
  const uint64_t nb = k / 256;
  for (uint64_t parts = 2; parts <= 8; ++parts) {
    if (nb % parts != 0) continue;
    float* part = reinterpret_cast<float*>(stream_scratch(st, parts * rows * n * 4, 3));
    if (part == nullptr) return kUnsupportedFeature;
    const int rc = staged(part, parts);
    if (rc == kUnsupportedFeature) continue;
    if (rc != kOk) return rc;
    return tsr_gemm_vec_reduce(part, c, rows * n, parts, st);
  }
  return kUnsupportedFeature;
}

}  // namespace

namespace tsr {
int gemm_q4k_dispatch(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                      uint64_t split, cudaStream_t st, bool allow_scratch) {
  // more than four rows: passes of eight (or four) rows; up to eight rows that is one pass wherever it fits
  const int rc = (m > kStagedRows / 2 && split == 1)
                     ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
                         int r = staged_gemm_q4k(a + i0 * k, w, c + i0 * n, rows, n, k, 1, st);
                         // (larger batches of such a k are faster on the tile, which cuts k among its CTAs: 55 against 69 us at m = 16)
                         if (r == kUnsupportedFeature && rows > kStagedRows / 2 && m <= kStagedRows && allow_scratch)
                           r = staged_pass_cut(rows, n, k, c + i0 * n, st, [&](float* part, uint64_t parts) {
                             return staged_gemm_q4k(a + i0 * k, w, part, rows, n, k, parts, st);
                           });
                         return r;
                       }, kStagedRows)
                     : staged_gemm_q4k(a, w, c, m, n, k, split, st);
  if (rc != kUnsupportedFeature) return rc;
  if (m >= 9 && split == 1) {
    const int rt = umma_gemm(0, a, w, nullptr, c, m, n, k, st, allow_scratch);
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_q4k(a, w, c, m, n, k, split, st);
}
}  // namespace tsr

extern "C" {

int tsr_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream) {
  if (!a || !w || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) || k % 256 != 0 ||
      split == 0 || (k / 256) % split != 0 || split > 65535)
    return kInvalidArgument;
  if (!aligned16(a) || !aligned16(w) || !aligned16(c)) return kInvalidArgument;
  return gemm_q4k_dispatch(a, w, c, m, n, k, split, static_cast<cudaStream_t>(stream), true);
}

int tsr_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream) {
  if (!a || !w || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) || k % 256 != 0 ||
      split == 0 || (k / 256) % split != 0 || split > 65535)
    return kInvalidArgument;
  if (!aligned16(a) || (reinterpret_cast<uintptr_t>(w) & 1u) || !aligned16(c))
    return kInvalidArgument;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = (m > kStagedRows / 2 && split == 1)
                     ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
                         int r = staged_gemm_q6k(a + i0 * k, w, c + i0 * n, rows, n, k, 1, st);
                         if (r == kUnsupportedFeature && rows > kStagedRows / 2)
                           r = staged_pass_cut(rows, n, k, c + i0 * n, st, [&](float* part, uint64_t parts) {
                             return staged_gemm_q6k(a + i0 * k, w, part, rows, n, k, parts, st);
                           });
                         return r;
                       }, kQ6KStagedRows)
                     : staged_gemm_q6k(a, w, c, m, n, k, split, st);
  if (rc != kUnsupportedFeature) return rc;
  if (m >= 2 && split == 1) {
    const int rt = umma_gemm(1, a, w, nullptr, c, m, n, k, static_cast<cudaStream_t>(stream));
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_q6k(a, w, c, m, n, k, split, static_cast<cudaStream_t>(stream));
}

int tsr_gemm_mxfp4(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                   void* stream) {
  if (!a || !w || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) || k % 32 != 0)
    return kInvalidArgument;
  if (!aligned16(a) || !aligned16(w) || !aligned16(c)) return kInvalidArgument;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // batches: nibbles and scales go from HBM to the tensor core without a thread touching a weight
    const int rt = umma_mxfp4_gemm(a, w, c, m, n, k, st);
    if (rt != kUnsupportedFeature) return rt;
  }
  const int rc = m > kStagedRows ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
    return staged_gemm_mxfp4(a + i0 * k, w, c + i0 * n, rows, n, k, st);
  }) : staged_gemm_mxfp4(a, w, c, m, n, k, st);
  if (rc != kUnsupportedFeature) return rc;
  if (m >= 2) {
    const int rt = umma_gemm(2, a, w, nullptr, c, m, n, k, static_cast<cudaStream_t>(stream));
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_mxfp4(a, w, c, m, n, k, static_cast<cudaStream_t>(stream));
}

int tsr_gemm_fp8(const float* a, const void* w, const float* s, float* c, uint64_t m, uint64_t n,
                 uint64_t k, void* stream) {
  if (!a || !w || !s || !c || !fits_int(m) || !fits_int(n) || !fits_int(k)) return kInvalidArgument;
  if (!aligned16(a) || !aligned16(w) || !aligned16(c)) return kInvalidArgument;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // batches: the weights go from HBM to the tensor core without a thread touching them
    const int rt = umma_f8_gemm(a, w, s, c, m, n, k, st);
    if (rt != kUnsupportedFeature) return rt;
  }
  const int rc = m > kStagedRows ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
    return staged_gemm_fp8(a + i0 * k, w, s, c + i0 * n, rows, n, k, st);
  }) : staged_gemm_fp8(a, w, s, c, m, n, k, st);
  if (rc != kUnsupportedFeature) return rc;
  if (m >= 2 && k % 64 == 0) {
    const int rt = umma_gemm(3, a, w, s, c, m, n, k, static_cast<cudaStream_t>(stream));
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_fp8(a, w, s, c, m, n, k, static_cast<cudaStream_t>(stream));
}

int tsr_gemm_mxfp4_w4a8(const void* a_fp8, const void* w, const float* as, const void* wref,
                        float* c, uint64_t m, uint64_t n, uint64_t k, uint64_t split,
                        void* stream) {
  if (!a_fp8 || !w || !as || !wref || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) ||
      k % 32 != 0 || split == 0 || split > 65535)
    return kInvalidArgument;
  if (!aligned16(a_fp8) || !aligned16(w) || !aligned16(c)) return kInvalidArgument;
  if (split == 1) {
    // Unsplit: the block-scaled tensor-core tile, E4M3 activation codes against the nibbles with
    // their own E8M0 scales.  The reference folds each weight into an E4M3 byte relative to the
    // row's largest scale first (FoldMxFp4ToFp8, src/core/numerics/quant.cpp:846-924), which is
    // exact while a block's scale is within 2^8 of that largest one and drops bits beyond; the
    // tile never drops them, so it equals the reference there and is closer to the unfolded
    // product elsewhere.  wref is not needed.
    const int rt = umma_mxfp4_w4a8(a_fp8, as, w, c, m, n, k, static_cast<cudaStream_t>(stream));
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_w4a8(a_fp8, w, as, wref, c, m, n, k, split, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ------------------------------------------------------------ name table

namespace {

struct Args {
  const void* const* buf;
  const size_t* bytes;
  int nbuf;
  const uint64_t* sc;
  int nsc;
  uint32_t grid_y;
  cudaStream_t stream;
  bool dry;          // check the arguments only (a deferred launch is checked when it is made)
  tsr_context* ctx;  // for the ids that need the context's scratch or communicator
};

bool shape(const Args& a, int nbuf, int nsc) { return a.nbuf == nbuf && a.nsc == nsc; }
bool holds(const Args& a, int i, uint64_t need) { return a.bytes[i] >= need; }

constexpr uint64_t kMaxDim = 0x7FFFFFFFull;
bool dims_ok(uint64_t m, uint64_t n, uint64_t k) {
  return m > 0 && n > 0 && k > 0 && m <= kMaxDim && n <= kMaxDim && k <= kMaxDim;
}

template <uint64_t BLOCK_BYTES, bool Q6>
int block_gemm(const Args& a, uint64_t split, uint64_t rows_required) {
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k) || k % 256 != 0 || split == 0 || (k / 256) % split != 0)
    return kInvalidArgument;
  if (rows_required != 0 && m != rows_required) return kInvalidArgument;
  if (a.grid_y != 0 && a.grid_y != split) return kInvalidArgument;
  if (!holds(a, 0, m * k * 4) || !holds(a, 1, n * (k / 256) * BLOCK_BYTES) ||
      !holds(a, 2, split * m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto* A = static_cast<const float*>(a.buf[0]);
  auto* C = static_cast<float*>(const_cast<void*>(a.buf[2]));
  return Q6 ? tsr_gemm_q6k(A, a.buf[1], C, m, n, k, split, a.stream)
            : tsr_gemm_q4k(A, a.buf[1], C, m, n, k, split, a.stream);
}

// gemm_q4k / gemm_q4k_row / gemm_q4k_batched / gemm_q4k_wmma: scalars m, n, k
// (include/tessera/backend.hpp:153-161,207-212; src/core/decode_internal.hpp:1466-1517).
template <uint64_t BB, bool Q6>
int k_block_plain(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  Args b = a;
  b.grid_y = 0;
  return block_gemm<BB, Q6>(b, 1, 0);
}
// gemm_q4k_vec / gemm_q6k_vec: scalars m, n, k, split
// (src/backends/vulkan/kernels/gemm_q4k_vec.comp:7-14).
template <uint64_t BB, bool Q6>
int k_block_vec(const Args& a) {
  if (!shape(a, 3, 4)) return kInvalidArgument;
  return block_gemm<BB, Q6>(a, a.sc[3], 0);
}
// gemm_q4k_rows<R>: scalars m, n, k, split with m == R
// (src/backends/vulkan/kernels/gemm_q4k_rows2.comp:7-12).
template <uint64_t BB, bool Q6, int R>
int k_block_rows(const Args& a) {
  if (!shape(a, 3, 4)) return kInvalidArgument;
  return block_gemm<BB, Q6>(a, a.sc[3], R);
}

// gemm_vec_reduce, gemm_mxfp4_wmma_reduce: buffers part, out; scalars total, split.
int k_vec_reduce(const Args& a) {
  if (!shape(a, 2, 2)) return kInvalidArgument;
  const uint64_t total = a.sc[0], split = a.sc[1];
  if (total == 0 || split == 0 || !holds(a, 0, split * total * 4) || !holds(a, 1, total * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_gemm_vec_reduce(static_cast<const float*>(a.buf[0]),
                             static_cast<float*>(const_cast<void*>(a.buf[1])), total, split,
                             a.stream);
}

// gemm_mxfp4 / gemm_mxfp4_rows / gemm_mxfp4_batched: scalars m, n, k
// (backend.hpp:195-201; gemm_mxfp4_rows.comp:3-6).
int k_mxfp4(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k) || k % 32 != 0) return kInvalidArgument;
  if (!holds(a, 0, m * k * 4) || !holds(a, 1, n * (k / 2) + n * (k / 32)) || !holds(a, 2, m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_gemm_mxfp4(static_cast<const float*>(a.buf[0]), a.buf[1],
                        static_cast<float*>(const_cast<void*>(a.buf[2])), m, n, k, a.stream);
}

// gemm_mxfp4_wmma: buffers A8, W, As, Wref, C; scalars m, n, k, split, wperm
// (src/backends/vulkan/kernels/gemm_mxfp4_wmma.comp:5-13).
int k_mxfp4_wmma(const Args& a) {
  if (!shape(a, 5, 5)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2], split = a.sc[3], wperm = a.sc[4];
  if (!dims_ok(m, n, k) || k % 32 != 0 || split == 0) return kInvalidArgument;
  if (wperm != 0) return kUnsupportedFeature;  // only the packed layout exists
  if (a.grid_y != 0 && a.grid_y != split) return kInvalidArgument;
  if (!holds(a, 0, m * k) || !holds(a, 1, n * (k / 2) + n * (k / 32)) || !holds(a, 2, m * 4) ||
      !holds(a, 3, n) || !holds(a, 4, split * m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_gemm_mxfp4_w4a8(a.buf[0], a.buf[1], static_cast<const float*>(a.buf[2]), a.buf[3],
                             static_cast<float*>(const_cast<void*>(a.buf[4])), m, n, k, split,
                             a.stream);
}

// mxfp4_row_ref: buffers W, Wref; scalars n, k (mxfp4_row_ref.comp:5-8).
int k_row_ref(const Args& a) {
  if (!shape(a, 2, 2)) return kInvalidArgument;
  const uint64_t n = a.sc[0], k = a.sc[1];
  if (!dims_ok(1, n, k) || k % 32 != 0) return kInvalidArgument;
  if (!holds(a, 0, n * (k / 2) + n * (k / 32)) || !holds(a, 1, n)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_mxfp4_row_ref(a.buf[0], const_cast<void*>(a.buf[1]), n, k, a.stream);
}

// gemm_fp8: buffers A, W, S, C; scalars m, n, k (backend.hpp:190-194).
int k_fp8(const Args& a) {
  if (!shape(a, 4, 3)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k)) return kInvalidArgument;
  if (!holds(a, 0, m * k * 4) || !holds(a, 1, n * k) || !holds(a, 2, n * 4) ||
      !holds(a, 3, m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_gemm_fp8(static_cast<const float*>(a.buf[0]), a.buf[1],
                      static_cast<const float*>(a.buf[2]),
                      static_cast<float*>(const_cast<void*>(a.buf[3])), m, n, k, a.stream);
}

// quantize_fp8: buffers data, scale; scalars rows, cols (backend.hpp:294-299).
int k_quant(const Args& a) {
  if (!shape(a, 2, 2)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1];
  if (!dims_ok(rows, cols, 1) || !holds(a, 0, rows * cols * 4) || !holds(a, 1, rows * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_quantize_fp8(static_cast<float*>(const_cast<void*>(a.buf[0])),
                          static_cast<float*>(const_cast<void*>(a.buf[1])), rows, cols, a.stream);
}

// quantize_fp8_pack / quantize_fp8_pack_rows: buffers in, codes, scale;
// scalars rows, cols (backend.hpp:302-307; quantize_fp8_pack_rows.comp:10-13).
int k_quant_pack(const Args& a) {
  if (!shape(a, 3, 2)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1];
  if (!dims_ok(rows, cols, 1) || cols % 4 != 0 || !holds(a, 0, rows * cols * 4) ||
      !holds(a, 1, rows * cols) || !holds(a, 2, rows * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_quantize_fp8_pack(static_cast<const float*>(a.buf[0]), const_cast<void*>(a.buf[1]),
                               static_cast<float*>(const_cast<void*>(a.buf[2])), rows, cols,
                               a.stream);
}

// round_bf16: buffer x; scalar n (backend.hpp:341-345).
int k_round(const Args& a) {
  if (!shape(a, 1, 1)) return kInvalidArgument;
  if (a.sc[0] == 0 || !holds(a, 0, a.sc[0] * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_round_bf16(static_cast<float*>(const_cast<void*>(a.buf[0])), a.sc[0], a.stream);
}

// add: buffers A, B, O; scalar n (backend.hpp:258-260).
int k_add(const Args& a) {
  if (!shape(a, 3, 1)) return kInvalidArgument;
  const uint64_t n = a.sc[0];
  if (n == 0 || !holds(a, 0, n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_add(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                 static_cast<float*>(const_cast<void*>(a.buf[2])), n, a.stream);
}

// silu_mul: buffers G, U, O; scalar n (backend.hpp:257-260).
int k_silu_mul(const Args& a) {
  if (!shape(a, 3, 1)) return kInvalidArgument;
  const uint64_t n = a.sc[0];
  if (n == 0 || !holds(a, 0, n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_silu_mul(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                      static_cast<float*>(const_cast<void*>(a.buf[2])), n, a.stream);
}

float float_of_bits(uint64_t v) {
  const uint32_t b = static_cast<uint32_t>(v);
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

// rmsnorm: buffers X, W, Y; scalars rows, cols, eps as fp32 bits (backend.hpp:212-216).
int k_rmsnorm(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1];
  const float eps = float_of_bits(a.sc[2]);
  if (!dims_ok(rows, cols, 1) || !(eps >= 0.0f) || !holds(a, 0, rows * cols * 4) || !holds(a, 1, cols * 4) ||
      !holds(a, 2, rows * cols * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_rmsnorm(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                     static_cast<float*>(const_cast<void*>(a.buf[2])), rows, cols, eps, a.stream);
}

// sigmoid_gate: buffers A, G, O; scalar n (backend.hpp:217-219).
int k_sigmoid_gate(const Args& a) {
  if (!shape(a, 3, 1)) return kInvalidArgument;
  const uint64_t n = a.sc[0];
  if (n == 0 || !holds(a, 0, n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, n * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_sigmoid_gate(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                          static_cast<float*>(const_cast<void*>(a.buf[2])), n, a.stream);
}

// l2norm: buffers X, Y; scalars rows, cols, eps bits, scale bits (backend.hpp:220-223).
int k_l2norm(const Args& a) {
  if (!shape(a, 2, 4)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1];
  const float eps = float_of_bits(a.sc[2]), scale = float_of_bits(a.sc[3]);
  if (!dims_ok(rows, cols, 1) || !(eps >= 0.0f) || !holds(a, 0, rows * cols * 4) || !holds(a, 1, rows * cols * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_l2norm(static_cast<const float*>(a.buf[0]), static_cast<float*>(const_cast<void*>(a.buf[1])), rows, cols, eps,
                    scale, a.stream);
}

// rmsnorm_gated: buffers X, W, gate, Y; scalars rows, cols, eps bits, gbase, ybase (backend.hpp:224-233).
int k_rmsnorm_gated(const Args& a) {
  if (!shape(a, 4, 5)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1], gbase = a.sc[3], ybase = a.sc[4];
  const float eps = float_of_bits(a.sc[2]);
  if (!dims_ok(rows, cols, 1) || !(eps >= 0.0f) || gbase > kMaxDim * 1024 || ybase > kMaxDim * 1024) return kInvalidArgument;
  if (!holds(a, 0, rows * cols * 4) || !holds(a, 1, cols * 4) || !holds(a, 2, (gbase + rows * cols) * 4) ||
      !holds(a, 3, (ybase + rows * cols) * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_rmsnorm_gated(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                           static_cast<const float*>(a.buf[2]), static_cast<float*>(const_cast<void*>(a.buf[3])), rows, cols,
                           eps, gbase, ybase, a.stream);
}

// ssm_gate: buffers a_log, dt (heads), alpha_raw, beta_raw, alpha, beta (rows x heads); scalars heads, rows
// (backend.hpp:234-238).
int k_ssm_gate(const Args& a) {
  if (!shape(a, 6, 2)) return kInvalidArgument;
  const uint64_t heads = a.sc[0], rows = a.sc[1];
  if (!dims_ok(heads, rows, 1) || !holds(a, 0, heads * 4) || !holds(a, 1, heads * 4)) return kInvalidArgument;
  for (int i = 2; i < 6; ++i)
    if (!holds(a, i, rows * heads * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_ssm_gate(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                      static_cast<const float*>(a.buf[2]), static_cast<const float*>(a.buf[3]),
                      static_cast<float*>(const_cast<void*>(a.buf[4])), static_cast<float*>(const_cast<void*>(a.buf[5])),
                      heads, rows, a.stream);
}

// qgate_split: buffers fused, Q, G; scalars heads, head_dim, rows (backend.hpp:386-390).
int k_qgate_split(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t heads = a.sc[0], dim = a.sc[1], rows = a.sc[2];
  if (!dims_ok(heads, dim, rows)) return kInvalidArgument;
  const uint64_t n = rows * heads * dim;
  if (!holds(a, 0, 2 * n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, n * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_qgate_split(static_cast<const float*>(a.buf[0]), static_cast<float*>(const_cast<void*>(a.buf[1])),
                         static_cast<float*>(const_cast<void*>(a.buf[2])), heads, dim, rows, a.stream);
}

// repeat_heads: buffers IN, OUT; scalars num_v_heads, head_k_dim, factor, rows (backend.hpp:249-254).
int k_repeat_heads(const Args& a) {
  if (!shape(a, 2, 4)) return kInvalidArgument;
  const uint64_t vh = a.sc[0], dim = a.sc[1], factor = a.sc[2], rows = a.sc[3];
  if (!dims_ok(vh, dim, rows) || factor == 0 || vh % factor != 0) return kInvalidArgument;
  if (!holds(a, 0, rows * (vh / factor) * dim * 4) || !holds(a, 1, rows * vh * dim * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_repeat_heads(static_cast<const float*>(a.buf[0]), static_cast<float*>(const_cast<void*>(a.buf[1])), vh, dim,
                          factor, rows, a.stream);
}

// embedding_f32 / _bf16 / _q4k: buffers ids (u32, rows), table (vocab x cols), out (fp32, rows x cols);
// scalars rows, cols, vocab (backend.hpp:261-265).
template <int KIND>
int k_embedding(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1], vocab = a.sc[2];
  if (!dims_ok(rows, cols, vocab) || (KIND == 2 && cols % 256 != 0)) return kInvalidArgument;
  const uint64_t table = KIND == 0 ? vocab * cols * 4 : KIND == 1 ? vocab * cols * 2 : vocab * (cols / 256) * 144;
  if (!holds(a, 0, rows * 4) || !holds(a, 1, table) || !holds(a, 2, rows * cols * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_embedding(KIND, static_cast<const uint32_t*>(a.buf[0]), a.buf[1], static_cast<float*>(const_cast<void*>(a.buf[2])),
                       rows, cols, vocab, a.stream);
}

// mrope: buffers io (rows x heads x head_dim), pos (rows x 3 u64); scalars rows, heads, head_dim, rope_dim,
// theta bits, sec_t, sec_h, sec_w (backend.hpp:378-385).
int k_mrope(const Args& a) {
  if (!shape(a, 2, 8)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], heads = a.sc[1], dim = a.sc[2], rdim = a.sc[3];
  if (!dims_ok(rows, heads, dim) || rdim == 0 || rdim > dim || dim % 2 != 0 || rdim % 2 != 0 ||
      a.sc[5] > rdim || a.sc[6] > rdim || a.sc[7] > rdim || a.sc[5] + a.sc[6] + a.sc[7] > rdim / 2)
    return kInvalidArgument;
  if (!holds(a, 0, rows * heads * dim * 4) || !holds(a, 1, rows * 3 * 8)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_mrope(static_cast<float*>(const_cast<void*>(a.buf[0])), static_cast<const uint64_t*>(a.buf[1]), rows, heads, dim,
                   rdim, float_of_bits(a.sc[4]), a.sc[5], a.sc[6], a.sc[7], a.stream);
}

// gemm_f32* / gemm_bf16*: buffers A, W, C; scalars m, n, k (backend.hpp:180-190).
template <int BF16>
int k_gemm_dense(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k) || !holds(a, 0, m * k * 4) || !holds(a, 1, n * k * (BF16 ? 2 : 4)) || !holds(a, 2, m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_gemm_dense(BF16, static_cast<const float*>(a.buf[0]), a.buf[1], static_cast<float*>(const_cast<void*>(a.buf[2])), m, n,
                        k, a.stream);
}

// rope: buffer io; scalars rows, heads, head_dim, rope_dim, pos_base, theta bits (backend.hpp:162-166).
int k_rope(const Args& a) {
  if (!shape(a, 1, 6)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], heads = a.sc[1], dim = a.sc[2], rdim = a.sc[3];
  if (!dims_ok(rows, heads, dim) || rdim == 0 || rdim > dim || dim % 2 != 0 || rdim % 2 != 0) return kInvalidArgument;
  if (!holds(a, 0, rows * heads * dim * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_rope(static_cast<float*>(const_cast<void*>(a.buf[0])), rows, heads, dim, rdim, a.sc[4], float_of_bits(a.sc[5]),
                  a.stream);
}

// quantize_q8 / quantize_q4: buffers In (fp32 rows x cols), codes, scale; scalars rows, cols (backend.hpp:283-298).
template <int KIND>
int k_quantize_rows(const Args& a) {
  if (!shape(a, 3, 2)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], cols = a.sc[1];
  if (!dims_ok(rows, cols, 1) || cols % (KIND == 0 ? 4 : 8) != 0 || !holds(a, 0, rows * cols * 4) ||
      !holds(a, 1, KIND == 0 ? rows * cols : rows * cols / 2) || !holds(a, 2, rows * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_quantize_rows(KIND, static_cast<const float*>(a.buf[0]), const_cast<void*>(a.buf[1]),
                           static_cast<float*>(const_cast<void*>(a.buf[2])), rows, cols, a.stream);
}

// cast_f32_f16: buffers In (fp32), Out (fp16); scalar n, even (backend.hpp:334-336).
int k_cast_f16(const Args& a) {
  if (!shape(a, 2, 1)) return kInvalidArgument;
  const uint64_t n = a.sc[0];
  if (n == 0 || n % 2 != 0 || !holds(a, 0, n * 4) || !holds(a, 1, n * 2)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_cast_f32_f16(static_cast<const float*>(a.buf[0]), const_cast<void*>(a.buf[1]), n, a.stream);
}

// delta_step_heads: buffers S, k, v, q, o, alpha, beta; scalars heads, dk, dv, rows, sbase, sstride, abase
// (backend.hpp:239-248).
int k_delta_step_heads(const Args& a) {
  if (!shape(a, 7, 7)) return kInvalidArgument;
  const uint64_t heads = a.sc[0], dk = a.sc[1], dv = a.sc[2], rows = a.sc[3], sbase = a.sc[4], sstride = a.sc[5], abase = a.sc[6];
  if (!dims_ok(heads, dk, dv) || rows == 0 || rows > kMaxDim || dk > 256 || sbase > kMaxDim * 1024 || sstride > kMaxDim * 1024 ||
      abase > kMaxDim * 1024)
    return kInvalidArgument;
  const uint64_t state = heads * dk * dv;
  const uint64_t s_need = sbase + (sstride == 0 ? state : rows * sstride + state);
  if (!holds(a, 0, s_need * 4) || !holds(a, 1, rows * heads * dk * 4) || !holds(a, 2, rows * heads * dv * 4) ||
      !holds(a, 3, rows * heads * dk * 4) || !holds(a, 4, rows * heads * dv * 4) ||
      !holds(a, 5, (abase + rows * heads) * 4) || !holds(a, 6, (abase + rows * heads) * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_delta_step_heads(static_cast<float*>(const_cast<void*>(a.buf[0])), static_cast<const float*>(a.buf[1]),
                              static_cast<const float*>(a.buf[2]), static_cast<const float*>(a.buf[3]),
                              static_cast<float*>(const_cast<void*>(a.buf[4])), static_cast<const float*>(a.buf[5]),
                              static_cast<const float*>(a.buf[6]), heads, dk, dv, rows, sbase, sstride, abase, a.stream);
}

// conv1d_state: buffers qkv, W (conv_dim x width), hist (conv_dim x (width-1)), q, k, v, hist_hist; scalars
// conv_dim, width, key_dim, qkv_offset, rows, hist_stride (src/backends/rocm/rocm_kernels.hpp:580-589).
int k_conv1d_state(const Args& a) {
  if (!shape(a, 7, 6)) return kInvalidArgument;
  const uint64_t cd = a.sc[0], width = a.sc[1], kd = a.sc[2], off = a.sc[3], rows = a.sc[4], hs = a.sc[5];
  if (!dims_ok(cd, width, rows) || 2 * kd > cd || off > kMaxDim * 1024 || hs > kMaxDim * 1024) return kInvalidArgument;
  const uint64_t hist = cd * (width - 1), vd = cd - 2 * kd;
  if (!holds(a, 0, (off + rows * cd) * 4) || !holds(a, 1, cd * width * 4) || !holds(a, 2, hist * 4) ||
      !holds(a, 3, rows * kd * 4) || !holds(a, 4, rows * kd * 4) || !holds(a, 5, rows * vd * 4) ||
      (hs != 0 && !holds(a, 6, (rows * hs + hist) * 4)))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto f = [&](int i) { return static_cast<float*>(const_cast<void*>(a.buf[i])); };
  return tsr_conv1d_state(f(0), f(1), f(2), f(3), f(4), f(5), f(6), cd, width, kd, off, rows, hs, a.stream);
}

// top_k_rows: buffers logits, ids (u32), vals; scalars rows, vocab, top_k, row_base
// (src/backends/rocm/rocm_kernels.hpp:558-566).
int k_top_k_rows(const Args& a) {
  if (!shape(a, 3, 4)) return kInvalidArgument;
  const uint64_t rows = a.sc[0], vocab = a.sc[1], top_k = a.sc[2], base = a.sc[3];
  if (!dims_ok(rows, vocab, top_k) || top_k > 32 || base > kMaxDim) return kInvalidArgument;
  if (!holds(a, 0, (base + rows) * vocab * 4) || !holds(a, 1, rows * top_k * 4) || !holds(a, 2, rows * top_k * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_top_k_rows(static_cast<const float*>(a.buf[0]), static_cast<uint32_t*>(const_cast<void*>(a.buf[1])),
                        static_cast<float*>(const_cast<void*>(a.buf[2])), rows, vocab, top_k, base, a.stream);
}

// attention: buffers q, k, v, out; scalars m, n, heads, kv_heads, head_dim, q_base, row_base, window, kv_f16, causal
// (backend.hpp:167-179).
bool attention_dims_ok(uint64_t m, uint64_t n, uint64_t heads, uint64_t kvh, uint64_t d, uint64_t rb, uint64_t win) {
  return dims_ok(m, n, heads) && dims_ok(kvh, d, 1) && heads % kvh == 0 && d <= 256 && rb <= kMaxDim && win <= kMaxDim;
}
// what the kernel serves (told before anything is queued): head_dim 128 or 256, at most 8 query heads per kv head
bool attention_served(uint64_t heads, uint64_t kvh, uint64_t d) { return (d == 128 || d == 256) && heads / kvh <= 8; }
uint64_t cache_bytes(int kv_format, uint64_t elems) {
  return kv_format == TSR_KV_F32 ? elems * 4 : kv_format == TSR_KV_F16 ? elems * 2 : kv_format == TSR_KV_INT4 ? elems / 2 : elems;
}
constexpr int kQuantKv[3] = {TSR_KV_INT8, TSR_KV_INT4, TSR_KV_FP8};  // the reference's `kind` 0, 1, 2

int k_attention(const Args& a) {
  if (!shape(a, 4, 10)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], heads = a.sc[2], kvh = a.sc[3], d = a.sc[4], qb = a.sc[5], rb = a.sc[6], win = a.sc[7];
  if (!attention_dims_ok(m, n, heads, kvh, d, rb, win)) return kInvalidArgument;
  if (!attention_served(heads, kvh, d)) return kUnsupportedFeature;
  const int fmt = a.sc[8] != 0 ? TSR_KV_F16 : TSR_KV_F32;
  if (!holds(a, 0, (rb + m) * heads * d * 4) || !holds(a, 1, cache_bytes(fmt, n * kvh * d)) ||
      !holds(a, 2, cache_bytes(fmt, n * kvh * d)) || !holds(a, 3, (rb + m) * heads * d * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_attention(fmt, static_cast<const float*>(a.buf[0]), a.buf[1], a.buf[2], nullptr, nullptr,
                       static_cast<float*>(const_cast<void*>(a.buf[3])), m, n, heads, kvh, d, qb, rb, win, a.sc[9], a.stream);
}

// attention_q8 / attention_q4 / attention_fp8: buffers q, k, v, k_scale, v_scale, out; scalars rows, n, heads,
// kv_heads, head_dim, q_base, row_base, window, kind (src/core/decode_internal.hpp:243-261; backend.hpp:283-309).
template <int KIND>
int k_attention_quant(const Args& a) {
  if (!shape(a, 6, 9)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], heads = a.sc[2], kvh = a.sc[3], d = a.sc[4], qb = a.sc[5], rb = a.sc[6], win = a.sc[7];
  if (!attention_dims_ok(m, n, heads, kvh, d, rb, win) || a.sc[8] != static_cast<uint64_t>(KIND)) return kInvalidArgument;
  if (!attention_served(heads, kvh, d)) return kUnsupportedFeature;
  const uint64_t cache = cache_bytes(kQuantKv[KIND], n * kvh * d);
  if (!holds(a, 0, (rb + m) * heads * d * 4) || !holds(a, 1, cache) || !holds(a, 2, cache) || !holds(a, 3, n * 4) ||
      !holds(a, 4, n * 4) || !holds(a, 5, (rb + m) * heads * d * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_attention(kQuantKv[KIND], static_cast<const float*>(a.buf[0]), a.buf[1], a.buf[2],
                       static_cast<const float*>(a.buf[3]), static_cast<const float*>(a.buf[4]),
                       static_cast<float*>(const_cast<void*>(a.buf[5])), m, n, heads, kvh, d, qb, rb, win, 1, a.stream);
}

// attention_split / attention_split_gqa: buffers q, k, v, pacc, pmax, psum; scalars rows, n, heads, kv_heads, head_dim,
// q_base, window, kv_f16, causal, split (src/core/decode_internal.hpp:317-343).  One kernel serves both ids: it always
// reads a key row once for all heads of its kv head.
int k_attention_split(const Args& a) {
  if (!shape(a, 6, 10)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], heads = a.sc[2], kvh = a.sc[3], d = a.sc[4], qb = a.sc[5], win = a.sc[6], split = a.sc[9];
  if (!attention_dims_ok(m, n, heads, kvh, d, 0, win) || split == 0 || split > 64) return kInvalidArgument;
  if (!attention_served(heads, kvh, d)) return kUnsupportedFeature;
  const int fmt = a.sc[7] != 0 ? TSR_KV_F16 : TSR_KV_F32;
  const uint64_t parts = m * heads * split;
  if (!holds(a, 0, m * heads * d * 4) || !holds(a, 1, cache_bytes(fmt, n * kvh * d)) ||
      !holds(a, 2, cache_bytes(fmt, n * kvh * d)) || !holds(a, 3, parts * d * 4) || !holds(a, 4, parts * 4) ||
      !holds(a, 5, parts * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto f = [&](int i) { return static_cast<float*>(const_cast<void*>(a.buf[i])); };
  return tsr_attention_split(fmt, f(0), a.buf[1], a.buf[2], nullptr, nullptr, f(3), f(4), f(5), m, n, heads, kvh, d, qb, win,
                             a.sc[8], split, a.stream);
}

// attention_q8_split / _q4_split / _fp8_split: buffers q, k, v, k_scale, v_scale, pacc, pmax, psum; scalars rows, n,
// heads, kv_heads, head_dim, q_base, window, kind, split (src/core/decode_internal.hpp:348-374).
template <int KIND>
int k_attention_quant_split(const Args& a) {
  if (!shape(a, 8, 9)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], heads = a.sc[2], kvh = a.sc[3], d = a.sc[4], qb = a.sc[5], win = a.sc[6], split = a.sc[8];
  if (!attention_dims_ok(m, n, heads, kvh, d, 0, win) || a.sc[7] != static_cast<uint64_t>(KIND) || split == 0 || split > 64)
    return kInvalidArgument;
  if (!attention_served(heads, kvh, d)) return kUnsupportedFeature;
  const uint64_t cache = cache_bytes(kQuantKv[KIND], n * kvh * d), parts = m * heads * split;
  if (!holds(a, 0, m * heads * d * 4) || !holds(a, 1, cache) || !holds(a, 2, cache) || !holds(a, 3, n * 4) ||
      !holds(a, 4, n * 4) || !holds(a, 5, parts * d * 4) || !holds(a, 6, parts * 4) || !holds(a, 7, parts * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto f = [&](int i) { return static_cast<float*>(const_cast<void*>(a.buf[i])); };
  return tsr_attention_split(kQuantKv[KIND], f(0), a.buf[1], a.buf[2], f(3), f(4), f(5), f(6), f(7), m, n, heads, kvh, d, qb, win,
                             1, split, a.stream);
}

// attention_combine: buffers pacc, pmax, psum, out; scalars rows, heads, head_dim, split
// (src/core/decode_internal.hpp:299-310).
int k_attention_combine(const Args& a) {
  if (!shape(a, 4, 4)) return kInvalidArgument;
  const uint64_t m = a.sc[0], heads = a.sc[1], d = a.sc[2], split = a.sc[3];
  if (!dims_ok(m, heads, d) || split == 0 || split > kMaxDim) return kInvalidArgument;
  const uint64_t parts = m * heads * split;
  if (!holds(a, 0, parts * d * 4) || !holds(a, 1, parts * 4) || !holds(a, 2, parts * 4) || !holds(a, 3, m * heads * d * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto f = [&](int i) { return static_cast<float*>(const_cast<void*>(a.buf[i])); };
  return tsr_attention_combine(f(0), f(1), f(2), f(3), m, heads, d, split, a.stream);
}

// fill: buffer int32; scalars value, count (backend.hpp:151-152).
int k_fill(const Args& a) {
  if (!shape(a, 1, 2)) return kInvalidArgument;
  const uint64_t n = a.sc[1];
  if (n == 0 || !holds(a, 0, n * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_fill(static_cast<int32_t*>(const_cast<void*>(a.buf[0])),
                  static_cast<int32_t>(a.sc[0]), n, a.stream);
}

// copy_d2d: buffers src, dst; scalars src_offset, dst_offset, bytes.  The queued form of a small device-to-device
// copy (the key / value rows a token appends to its cache, src/core/decode_internal.hpp:520-640 of the reference):
// a copy that flushed the queue would cut a token's launches into one piece per attention layer.
__global__ void copy_bytes_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, size_t bytes,
                                  int wide) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x, threads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (wide) {
    for (size_t i = tid; i < bytes / 16; i += threads) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (size_t i = tid; i < bytes; i += threads) dst[i] = src[i];
  }
}

int k_copy_d2d(const Args& a) {
  if (!shape(a, 2, 3)) return kInvalidArgument;
  const uint64_t so = a.sc[0], d_o = a.sc[1], bytes = a.sc[2];
  if (bytes == 0 || bytes > kQueuedCopyLimit || so > (1ull << 48) || d_o > (1ull << 48) || !holds(a, 0, so + bytes) ||
      !holds(a, 1, d_o + bytes))
    return kInvalidArgument;
  if (a.dry) return kOk;
  const unsigned char* src = static_cast<const unsigned char*>(a.buf[0]) + so;
  unsigned char* dst = static_cast<unsigned char*>(const_cast<void*>(a.buf[1])) + d_o;
  const bool wide = bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  // what it writes is registered, so that a launch which reads these bytes as weights ahead of its wait is held back
  const void* out = dst;
  const size_t out_bytes = bytes;
  pdl_allowed_ranges(a.stream, nullptr, nullptr, 0, &out, &out_bytes, 1);
  const size_t items = wide ? bytes / 16 : bytes;
  const unsigned blocks = static_cast<unsigned>(items / 256 + 1 < 592 ? items / 256 + 1 : 592);
  copy_bytes_kernel<<<blocks, 256, 0, a.stream>>>(src, dst, bytes, wide ? 1 : 0);
  return check_launch();
}

// Sum over tensor-parallel ranks of an [m][n] fp32 matrix in place, on the communicator
// bound to the context (tsr_tp_bind).  With one rank (or none bound) it is the identity.
int tp_sum_in_place(const Args& a, float* data, uint64_t m, uint64_t n) {
  if (a.ctx == nullptr || a.ctx->tp == nullptr) return kOk;
  return tp_allreduce_matrix(a.ctx->tp, data, m, n, a.stream);
}

// One or several projections that share A as one staged launch which splits k as it
// sees fit, adds the chunks itself and, with `tp`, ends with the sum over ranks.
// fmt: 0 Q4_K, 1 Q6_K.  kUnsupportedFeature: the caller issues the pieces one by one.
int fused_group(tsr_context* ctx, int fmt, const float* a, const GroupTarget* t, int count, uint64_t m, uint64_t k,
                bool with_tp, cudaStream_t st, const Prologue* pro = nullptr) {
  if (ctx == nullptr) return kUnsupportedFeature;
  // the staged kernels move activations, outputs and the folded steps' vectors 16 bytes at a time
  if (!aligned16(a) || (pro != nullptr && (!aligned16(pro->other) || !aligned16(pro->out)))) return kUnsupportedFeature;
  for (int i = 0; i < count; ++i)
    if (!aligned16(t[i].w) || !aligned16(t[i].c) || !aligned16(t[i].add_src) || !aligned16(t[i].add_out))
      return kUnsupportedFeature;
  TpTail tail{};
  const TpTail* tp = nullptr;
  if (with_tp && ctx->tp != nullptr) {
    if (int rc = tp_tail_of(ctx->tp, &tail)) return rc;
    // TSR_TP_FUSED=0 (experiments): the projection and the sum over ranks as two launches
    static const bool fused = [] {
      const char* v = std::getenv("TSR_TP_FUSED");
      return v == nullptr || std::atoi(v) != 0;
    }();
    if (tail.world > 1 && !fused) return kUnsupportedFeature;
    if (tail.world > 1) tp = &tail;
  }
  return fmt == 0 ? staged_group_q4k(a, t, count, m, k, 0, &ctx->scratch, tp, st, pro)
                  : staged_group_q6k(a, t, count, m, k, 0, &ctx->scratch, tp, st, pro);
}

// gemm_q4k_vec_allreduce / gemm_q6k_vec_allreduce: buffers A, W, C; scalars m, n, k.
// Row-parallel projection of this rank's k range followed by the sum over the ranks of
// the bound communicator; C receives the same bits on every rank.  No reference id:
// there the projection is followed by TpReduce (src/models/qwen3_5/trunk.cpp:226-266).
template <uint64_t BLOCK_BYTES, bool Q6>
int k_block_allreduce(const Args& a) {
  if (!shape(a, 3, 3)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k) || k % 256 != 0) return kInvalidArgument;
  if (!holds(a, 0, m * k * 4) || !holds(a, 1, n * (k / 256) * BLOCK_BYTES) || !holds(a, 2, m * n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  auto* A = static_cast<const float*>(a.buf[0]);
  auto* C = static_cast<float*>(const_cast<void*>(a.buf[2]));
  const GroupTarget t{a.buf[1], C, n};
  const int rc = fused_group(a.ctx, Q6 ? 1 : 0, A, &t, 1, m, k, true, a.stream);
  if (rc != kUnsupportedFeature) return rc;
  // outside the staged kernels' range: the projection by itself, then the same tiles' sum
  const int rp = Q6 ? tsr_gemm_q6k(A, a.buf[1], C, m, n, k, 1, a.stream) : tsr_gemm_q4k(A, a.buf[1], C, m, n, k, 1, a.stream);
  if (rp != kOk) return rp;
  return tp_sum_in_place(a, C, m, n);
}

// allreduce_sum: buffer X; scalars m, n.  X[m][n] becomes its sum over the ranks of the
// bound communicator (the job of TpReduce, trunk.cpp:226-266, for callers that keep
// their own projection launches).
int k_allreduce_sum(const Args& a) {
  if (!shape(a, 1, 2)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1];
  if (!dims_ok(m, n, 1) || !holds(a, 0, m * n * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tp_sum_in_place(a, static_cast<float*>(const_cast<void*>(a.buf[0])), m, n);
}

// gemm_<q4k|q6k|mxfp4|fp8>_bf16: the projection with bf16 storage on both sides.  Buffers A
// (bf16, m x k), W, [S for fp8], C (bf16, m x n); scalars m, n, k.  C = RoundBf16(sum in fp32)
// (RoundBf16Ref, src/core/numerics/quant.cpp:231-243), the sums being those of the fp32 id on
// the same values.  No reference id: there activations and outputs are fp32
// (include/tessera/backend.hpp:153-156) and round_bf16 is a pass of its own.
// FMT: 0 Q4_K, 1 Q6_K, 2 MXFP4, 3 FP8.
template <int FMT>
int k_gemm_bf16(const Args& a) {
  constexpr int kBufs = FMT == 3 ? 4 : 3;
  if (!shape(a, kBufs, 3)) return kInvalidArgument;
  const uint64_t m = a.sc[0], n = a.sc[1], k = a.sc[2];
  if (!dims_ok(m, n, k)) return kInvalidArgument;
  if ((FMT <= 1 && k % 256 != 0) || (FMT == 2 && k % 32 != 0) || k % 8 != 0) return kInvalidArgument;
  const uint64_t w_bytes = FMT == 0 ? n * (k / 256) * 144 : FMT == 1 ? n * (k / 256) * 210 : FMT == 2 ? n * (k / 2) + n * (k / 32) : n * k;
  if (!holds(a, 0, m * k * 2) || !holds(a, 1, w_bytes) || !holds(a, kBufs - 1, m * n * 2)) return kInvalidArgument;
  if (FMT == 3 && !holds(a, 2, n * 4)) return kInvalidArgument;
  if (!aligned16(a.buf[0]) || !aligned16(a.buf[kBufs - 1])) return kInvalidArgument;
  if (a.dry) return kOk;
  void* C = const_cast<void*>(a.buf[kBufs - 1]);
  if (FMT <= 1 && m <= 8) {
    // the staged kernels read and write bf16 themselves
    Prologue io{};
    io.bf16_in = io.bf16_out = true;
    const GroupTarget t{a.buf[1], static_cast<float*>(C), n};
    const int rc = fused_group(a.ctx, FMT, static_cast<const float*>(a.buf[0]), &t, 1, m, k, false, a.stream, &io);
    if (rc != kUnsupportedFeature) return rc;
  }
  // elsewhere: fp32 copies of A and C around the fp32 projection
  const size_t a_bytes = (m * k * 4 + 255) / 256 * 256;
  unsigned char* scratch = stream_scratch(a.stream, a_bytes + m * n * 4, 1);
  if (scratch == nullptr) return kUnsupportedFeature;
  float* a32 = reinterpret_cast<float*>(scratch);
  float* c32 = reinterpret_cast<float*>(scratch + a_bytes);
  if (int rc = convert_bf16_to_f32(a.buf[0], a32, m * k, a.stream)) return rc;
  int rc;
  if (FMT == 0) rc = tsr_gemm_q4k(a32, a.buf[1], c32, m, n, k, 1, a.stream);
  else if (FMT == 1) rc = tsr_gemm_q6k(a32, a.buf[1], c32, m, n, k, 1, a.stream);
  else if (FMT == 2) rc = tsr_gemm_mxfp4(a32, a.buf[1], c32, m, n, k, a.stream);
  else rc = tsr_gemm_fp8(a32, a.buf[1], static_cast<const float*>(a.buf[2]), c32, m, n, k, a.stream);
  if (rc != kOk) return rc;
  return convert_f32_to_bf16(c32, C, m * n, a.stream);
}

// moe_gate: buffers vals (top_k), x (hidden), w (hidden), wts (top_k), sig (1); scalars top_k, hidden
// (src/backends/rocm/rocm_kernels.hpp:604-612).
int k_moe_gate(const Args& a) {
  if (!shape(a, 5, 2)) return kInvalidArgument;
  const uint64_t top_k = a.sc[0], hidden = a.sc[1];
  if (!dims_ok(top_k, hidden, 1) || !holds(a, 0, top_k * 4) || !holds(a, 1, hidden * 4) || !holds(a, 2, hidden * 4) ||
      !holds(a, 3, top_k * 4) || !holds(a, 4, 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_moe_gate(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                      static_cast<const float*>(a.buf[2]), static_cast<float*>(const_cast<void*>(a.buf[3])),
                      static_cast<float*>(const_cast<void*>(a.buf[4])), top_k, hidden, a.stream);
}

// moe_scale_add: buffers a, b, f, o; scalars n, idx: o = a + f[idx] * b (rocm_kernels.hpp:613-617).
int k_moe_scale_add(const Args& a) {
  if (!shape(a, 4, 2)) return kInvalidArgument;
  const uint64_t n = a.sc[0], idx = a.sc[1];
  if (n == 0 || idx > kMaxDim || !holds(a, 0, n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, (idx + 1) * 4) ||
      !holds(a, 3, n * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_moe_scale_add(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                           static_cast<const float*>(a.buf[2]), static_cast<float*>(const_cast<void*>(a.buf[3])), n, idx,
                           a.stream);
}

// moe_experts_gate_up_q4k: buffers x (hidden), gate, up (3-D Q4_K: experts x inter rows), ids (top_k u32),
// phi (top_k x inter); scalars hidden, inter, top_k, gate_stride, up_stride (bytes per expert)
// (rocm_kernels.hpp:618-627).  The number of experts is what the weight buffers hold.
int k_moe_gate_up(const Args& a) {
  if (!shape(a, 5, 5)) return kInvalidArgument;
  const uint64_t hidden = a.sc[0], inter = a.sc[1], top_k = a.sc[2], gs = a.sc[3], us = a.sc[4];
  if (!dims_ok(hidden, inter, top_k) || hidden % 256 != 0) return kInvalidArgument;
  const uint64_t per = inter * (hidden / 256) * 144;
  if (gs < per || us < per) return kInvalidArgument;
  const uint64_t eg = (a.bytes[1] - per) / gs + 1, eu = (a.bytes[2] - per) / us + 1;
  if (a.bytes[1] < per || a.bytes[2] < per) return kInvalidArgument;
  if (!holds(a, 0, hidden * 4) || !holds(a, 3, top_k * 4) || !holds(a, 4, top_k * inter * 4)) return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_moe_experts_gate_up_q4k(static_cast<const float*>(a.buf[0]), a.buf[1], a.buf[2],
                                     static_cast<const uint32_t*>(a.buf[3]), static_cast<float*>(const_cast<void*>(a.buf[4])),
                                     hidden, inter, top_k, gs, us, eg < eu ? eg : eu, a.stream);
}

// moe_experts_down_q4k / _q6k: buffers phi (top_k x inter), down (3-D: experts x hidden rows), ids, wts
// (top_k), out (hidden); scalars hidden, inter, top_k, down_stride, accumulate
// (rocm_kernels.hpp:628-640; src/models/qwen3_5/moe.cpp:414-421).
template <int FMT>
int k_moe_down(const Args& a) {
  if (!shape(a, 5, 5)) return kInvalidArgument;
  const uint64_t hidden = a.sc[0], inter = a.sc[1], top_k = a.sc[2], ds = a.sc[3], accumulate = a.sc[4];
  if (!dims_ok(hidden, inter, top_k) || inter % 256 != 0) return kInvalidArgument;
  const uint64_t per = hidden * (inter / 256) * (FMT == 0 ? 144 : 210);
  if (ds < per || a.bytes[1] < per) return kInvalidArgument;
  const uint64_t experts = (a.bytes[1] - per) / ds + 1;
  if (!holds(a, 0, top_k * inter * 4) || !holds(a, 2, top_k * 4) || !holds(a, 3, top_k * 4) || !holds(a, 4, hidden * 4))
    return kInvalidArgument;
  if (a.dry) return kOk;
  return tsr_moe_experts_down(FMT, static_cast<const float*>(a.buf[0]), a.buf[1], static_cast<const uint32_t*>(a.buf[2]),
                              static_cast<const float*>(a.buf[3]), static_cast<float*>(const_cast<void*>(a.buf[4])), hidden,
                              inter, top_k, ds, accumulate, experts, a.stream);
}

struct Entry {
  const char* name;
  int (*fn)(const Args&);
};

const Entry kTable[] = {
    {"fill", k_fill},
    {"add", k_add},
    {"silu_mul", k_silu_mul},
    {"rmsnorm", k_rmsnorm},
    {"sigmoid_gate", k_sigmoid_gate},
    {"l2norm", k_l2norm},
    {"rmsnorm_gated", k_rmsnorm_gated},
    {"ssm_gate", k_ssm_gate},
    {"qgate_split", k_qgate_split},
    {"repeat_heads", k_repeat_heads},
    {"conv1d_state", k_conv1d_state},
    {"top_k_rows", k_top_k_rows},
    {"attention", k_attention},
    {"attention_q8", k_attention_quant<0>},
    {"attention_q4", k_attention_quant<1>},
    {"attention_fp8", k_attention_quant<2>},
    {"attention_split", k_attention_split},
    {"attention_split_gqa", k_attention_split},
    {"attention_q8_split", k_attention_quant_split<0>},
    {"attention_q4_split", k_attention_quant_split<1>},
    {"attention_fp8_split", k_attention_quant_split<2>},
    {"attention_combine", k_attention_combine},
    {"copy_d2d", k_copy_d2d},
    {"mrope", k_mrope},
    {"rope", k_rope},
    {"gemm_f32", k_gemm_dense<0>},
    {"gemm_f32_batched", k_gemm_dense<0>},
    {"gemm_bf16", k_gemm_dense<1>},
    {"gemm_bf16_batched", k_gemm_dense<1>},
    {"gemm_bf16_wmma", k_gemm_dense<1>},
    {"gemm_bf16_rows", k_gemm_dense<1>},
    {"quantize_q8", k_quantize_rows<0>},
    {"quantize_q4", k_quantize_rows<1>},
    {"cast_f32_f16", k_cast_f16},
    {"delta_step_heads", k_delta_step_heads},
    {"embedding_f32", k_embedding<0>},
    {"embedding_bf16", k_embedding<1>},
    {"embedding_q4k", k_embedding<2>},
    {"round_bf16", k_round},
    {"gemm_q4k", k_block_plain<144, false>},
    {"gemm_q4k_row", k_block_plain<144, false>},
    {"gemm_q4k_vec", k_block_vec<144, false>},
    {"gemm_q4k_rows2", k_block_rows<144, false, 2>},
    {"gemm_q4k_rows3", k_block_rows<144, false, 3>},
    {"gemm_q4k_rows4", k_block_rows<144, false, 4>},
    {"gemm_q4k_rows5", k_block_rows<144, false, 5>},
    {"gemm_q4k_batched", k_block_plain<144, false>},
    {"gemm_q4k_wmma", k_block_plain<144, false>},
    {"gemm_q6k", k_block_plain<210, true>},
    {"gemm_q6k_vec", k_block_vec<210, true>},
    {"gemm_q6k_rows2", k_block_rows<210, true, 2>},
    {"gemm_q6k_rows3", k_block_rows<210, true, 3>},
    {"gemm_q6k_rows4", k_block_rows<210, true, 4>},
    {"gemm_q6k_rows5", k_block_rows<210, true, 5>},
    {"gemm_q6k_batched", k_block_plain<210, true>},
    {"gemm_q6k_wmma", k_block_plain<210, true>},
    {"gemm_vec_reduce", k_vec_reduce},
    {"gemm_mxfp4", k_mxfp4},
    {"gemm_mxfp4_rows", k_mxfp4},
    {"gemm_mxfp4_batched", k_mxfp4},
    {"gemm_mxfp4_wmma", k_mxfp4_wmma},
    {"gemm_mxfp4_wmma_reduce", k_vec_reduce},
    {"mxfp4_row_ref", k_row_ref},
    {"gemm_fp8", k_fp8},
    {"quantize_fp8", k_quant},
    {"quantize_fp8_pack", k_quant_pack},
    {"quantize_fp8_pack_rows", k_quant_pack},
    {"gemm_q4k_vec_allreduce", k_block_allreduce<144, false>},
    {"gemm_q6k_vec_allreduce", k_block_allreduce<210, true>},
    {"allreduce_sum", k_allreduce_sum},
    {"moe_gate", k_moe_gate},
    {"moe_scale_add", k_moe_scale_add},
    {"moe_experts_gate_up_q4k", k_moe_gate_up},
    {"moe_experts_down_q4k", k_moe_down<0>},
    {"moe_experts_down_q6k", k_moe_down<1>},
    {"gemm_q4k_bf16", k_gemm_bf16<0>},
    {"gemm_q6k_bf16", k_gemm_bf16<1>},
    {"gemm_mxfp4_bf16", k_gemm_bf16<2>},
    {"gemm_fp8_bf16", k_gemm_bf16<3>},
};
constexpr int kCount = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));

}  // namespace

// ------------------------------------------------- deferred submission
//
// In deferred mode tsr_launch only queues.  When the queue is flushed (a copy, a
// synchronisation, tsr_flush) it is rewritten before it is issued:
//   * gemm_<q4k|q6k>_vec / _rows<R> with a split followed by the gemm_vec_reduce of
//     its partial buffer becomes one projection that writes the final output (the
//     launch picks its own split of k and adds the chunks itself; the caller's partial
//     buffer is then not written);
//   * consecutive projections of one format that read the same activations with the
//     same m and k become one launch over up to four weight tensors;
//   * a silu_mul or rmsnorm whose output is the activation matrix of the projection(s)
//     queued right after it is folded into that launch's activation staging (the output
//     buffer is still written, later readers find it);
//   * an add that follows a single projection (with or without the sum over ranks) and
//     takes its output as one operand is folded into that launch's output stage (the
//     projection's own output buffer is still written).
// Everything else is issued as it was queued, in order.  A rewritten queue that has
// been flushed before is replayed as a CUDA graph (captured on its second appearance,
// keyed by a hash of the queue as the caller made it).
namespace {

struct Projection {
  int fmt;  // 0 Q4_K, 1 Q6_K
  const float* a;
  GroupTarget t;
  uint64_t m, k;
  size_t ops;    // queue entries it stands for: 1, or 2 with the reduce
  bool with_tp;  // an _allreduce id
};

bool name_starts(const char* name, const char* prefix) { return std::strncmp(name, prefix, std::strlen(prefix)) == 0; }
bool name_ends(const char* name, const char* suffix) {
  const size_t a = std::strlen(name), b = std::strlen(suffix);
  return a >= b && std::strcmp(name + a - b, suffix) == 0;
}
bool is_named(const PendingLaunch& op, const char* name) { return std::strcmp(kTable[op.kernel].name, name) == 0; }

bool as_projection(const std::vector<PendingLaunch>& q, size_t i, Projection* out) {
  if (i >= q.size()) return false;
  const PendingLaunch& op = q[i];
  const char* name = kTable[op.kernel].name;
  int fmt;
  if (name_starts(name, "gemm_q4k")) fmt = 0;
  else if (name_starts(name, "gemm_q6k")) fmt = 1;
  else return false;
  if (op.nbuf != 3 || (op.nsc != 3 && op.nsc != 4)) return false;
  const bool with_tp = name_ends(name, "_allreduce");
  const uint64_t m = op.sc[0], n = op.sc[1], k = op.sc[2], split = op.nsc == 4 ? op.sc[3] : 1;
  // nine to sixteen rows (a verify step): two passes of the merged launch, see issue_queue
  if (m > 2 * kStagedRows || (m > kStagedRows && with_tp)) return false;
  *out = Projection{fmt, static_cast<const float*>(op.buf[0]),
                    GroupTarget{op.buf[1], static_cast<float*>(const_cast<void*>(op.buf[2])), n}, m, k, 1, with_tp};
  if (split == 1) return true;
  if (i + 1 >= q.size()) return false;
  const PendingLaunch& red = q[i + 1];
  if (!is_named(red, "gemm_vec_reduce") || red.buf[0] != op.buf[2] || red.sc[0] != m * n || red.sc[1] != split)
    return false;
  out->t.c = static_cast<float*>(const_cast<void*>(red.buf[1]));
  out->ops = 2;
  return true;
}

bool overlaps(const void* p, size_t pb, const void* q, size_t qb) {
  const auto* a = static_cast<const unsigned char*>(p);
  const auto* b = static_cast<const unsigned char*>(q);
  return a < b + qb && b < a + pb;
}

// TSR_FUSE_ELEMENTWISE=0 (experiments): silu_mul, rmsnorm and add stay launches of their own
bool fuse_elementwise() {
  static const bool on = [] {
    const char* v = std::getenv("TSR_FUSE_ELEMENTWISE");
    return v == nullptr || std::atoi(v) != 0;
  }();
  return on;
}

// q[i] as a step that can run inside the activation staging of the projection after it.
bool as_prologue(const tsr_context* ctx, const std::vector<PendingLaunch>& q, size_t i, Prologue* pro, const float** in,
                 uint64_t* rows, uint64_t* cols) {
  if (!ctx->fold_elementwise || !fuse_elementwise() || i + 1 >= q.size()) return false;
  const PendingLaunch& op = q[i];
  Projection next;
  if (!as_projection(q, i + 1, &next) || next.m > kStagedRows) return false;
  if (is_named(op, "silu_mul")) {
    const size_t bytes = op.sc[0] * 4;
    if (next.a != op.buf[2] || next.m * next.k != op.sc[0]) return false;
    // every CTA that stages the activations evaluates the step for all of them: with many
    // row tiles and a long k a kernel of its own is cheaper (measured: 107 CTAs x 17408
    // elements cost 2.5-8 us inside the launch, about 3 us as a launch)
    // ... and inside a launch that ends with the sum over ranks it measured slower than its own kernel at every
    // world size (per step of 64 layers: 3.89 against 3.57 ms on 2 GPUs, 3.20 against 2.97 ms on 4)
    if (next.with_tp) return false;
    const uint64_t repeated = ((next.t.n + 47) / 48) * next.m * next.k;
    static const uint64_t limit = [] {
      const char* v = std::getenv("TSR_FOLD_SILU_LIMIT");
      return v ? static_cast<uint64_t>(std::atoll(v)) : 1000000ull;
    }();
    if (repeated > limit) return false;
    if (overlaps(op.buf[2], bytes, op.buf[0], bytes) || overlaps(op.buf[2], bytes, op.buf[1], bytes)) return false;
    *pro = Prologue{kProSiluMul, static_cast<const float*>(op.buf[1]), static_cast<float*>(const_cast<void*>(op.buf[2])), 0.0f};
    *in = static_cast<const float*>(op.buf[0]);
    *rows = next.m;
    *cols = next.k;
    return true;
  }
  if (is_named(op, "rmsnorm")) {
    const uint64_t r = op.sc[0], c = op.sc[1];
    const size_t bytes = r * c * 4;
    if (next.a != op.buf[2] || next.m != r || next.k != c || c % 4 != 0) return false;
    if (overlaps(op.buf[2], bytes, op.buf[0], bytes) || overlaps(op.buf[2], bytes, op.buf[1], c * 4)) return false;
    *pro = Prologue{kProRmsNorm, static_cast<const float*>(op.buf[1]), static_cast<float*>(const_cast<void*>(op.buf[2])),
                    float_of_bits(op.sc[2])};
    *in = static_cast<const float*>(op.buf[0]);
    *rows = r;
    *cols = c;
    return true;
  }
  return false;
}

// q[i] as an add that can run in the output stage of the single projection `p` before it.
bool as_epilogue_add(const tsr_context* ctx, const std::vector<PendingLaunch>& q, size_t i, const Projection& p,
                     const float* act, size_t act_bytes, const Prologue* pro, GroupTarget* t) {
  if (!ctx->fold_elementwise || !fuse_elementwise() || i >= q.size() || !is_named(q[i], "add")) return false;
  const PendingLaunch& op = q[i];
  const size_t bytes = p.m * p.t.n * 4;
  if (op.sc[0] != p.m * p.t.n) return false;
  const void* other;
  if (op.buf[0] == p.t.c) other = op.buf[1];
  else if (op.buf[1] == p.t.c) other = op.buf[0];
  else return false;
  const void* o = op.buf[2];
  if (overlaps(other, bytes, p.t.c, bytes)) return false;
  if (o != other && overlaps(o, bytes, other, bytes)) return false;
  if (o != p.t.c && overlaps(o, bytes, p.t.c, bytes)) return false;
  if (overlaps(o, bytes, act, act_bytes)) return false;
  if (pro != nullptr) {
    if (overlaps(o, bytes, pro->other, act_bytes)) return false;
    if (pro->out != nullptr && overlaps(o, bytes, pro->out, act_bytes)) return false;
  }
  t->add_src = static_cast<const float*>(other);
  t->add_out = static_cast<float*>(const_cast<void*>(o));
  return true;
}

// ---- neighbouring small steps of a token that one kernel serves (launch.h: merged small steps).  Each matcher
// checks that the launches at q[i...] are exactly the sequence the reference's layer issues on the same buffers,
// issues the merged kernel and returns how many launches it stood for (0: not this pattern).

float* fbuf(const PendingLaunch& op, int i) { return static_cast<float*>(const_cast<void*>(op.buf[i])); }

// ssm_gate, conv1d_state, l2norm(q), l2norm(k), repeat_heads(q), repeat_heads(k)
// (src/models/qwen3_5/trunk.cpp:748-766 of the reference)
size_t merged_linear_mixer_inputs(tsr_context* ctx, const std::vector<PendingLaunch>& q, size_t i, int* rc) {
  if (!ctx->fold_elementwise || !fuse_elementwise() || i + 6 > q.size()) return 0;
  const PendingLaunch &gate = q[i], &conv = q[i + 1], &lq = q[i + 2], &lk = q[i + 3], &rq = q[i + 4], &rk = q[i + 5];
  if (!is_named(gate, "ssm_gate") || !is_named(conv, "conv1d_state") || !is_named(lq, "l2norm") || !is_named(lk, "l2norm") ||
      !is_named(rq, "repeat_heads") || !is_named(rk, "repeat_heads"))
    return 0;
  const uint64_t conv_dim = conv.sc[0], width = conv.sc[1], key_dim = conv.sc[2];
  if (gate.sc[1] != 1 || conv.sc[4] != 1 || conv.sc[5] != 0 || width == 0 || width > 64) return 0;
  const uint64_t k_heads = lq.sc[0], cols = lq.sc[1];
  if (lk.sc[0] != k_heads || lk.sc[1] != cols || k_heads * cols != key_dim || conv_dim % cols != 0 || cols % 32 != 0 || cols > 1024)
    return 0;
  if (lq.buf[0] != conv.buf[3] || lq.buf[1] != lq.buf[0] || lk.buf[0] != conv.buf[4] || lk.buf[1] != lk.buf[0]) return 0;
  const uint64_t v_heads = rq.sc[0], factor = rq.sc[2];
  if (rq.sc[1] != cols || rk.sc[1] != cols || rk.sc[0] != v_heads || rk.sc[2] != factor || rq.sc[3] != 1 || rk.sc[3] != 1 ||
      factor == 0 || v_heads != k_heads * factor || rq.buf[0] != conv.buf[3] || rk.buf[0] != conv.buf[4])
    return 0;
  // the expanded heads and the gate outputs must be buffers of their own
  const size_t exp_bytes = v_heads * cols * 4;
  for (const PendingLaunch* r : {&rq, &rk})
    if (overlaps(r->buf[1], exp_bytes, conv.buf[0], conv.bytes[0]) || overlaps(r->buf[1], exp_bytes, conv.buf[2], conv.bytes[2]) ||
        overlaps(r->buf[1], exp_bytes, conv.buf[3], key_dim * 4) || overlaps(r->buf[1], exp_bytes, conv.buf[4], key_dim * 4))
      return 0;
  if (overlaps(rq.buf[1], exp_bytes, rk.buf[1], exp_bytes)) return 0;
  for (int o = 4; o <= 5; ++o)
    if (overlaps(gate.buf[o], gate.sc[0] * 4, conv.buf[0], conv.bytes[0]) || overlaps(gate.buf[o], gate.sc[0] * 4, conv.buf[2], conv.bytes[2]))
      return 0;
  LinearMixerInputs p{};
  p.a_log = fbuf(gate, 0), p.dt = fbuf(gate, 1), p.alpha_raw = fbuf(gate, 2), p.beta_raw = fbuf(gate, 3);
  p.alpha = fbuf(gate, 4), p.beta = fbuf(gate, 5), p.gate_heads = static_cast<int>(gate.sc[0]);
  p.qkv = fbuf(conv, 0), p.conv_w = fbuf(conv, 1), p.hist = fbuf(conv, 2), p.q = fbuf(conv, 3), p.k = fbuf(conv, 4), p.v = fbuf(conv, 5);
  p.conv_dim = static_cast<int>(conv_dim), p.width = static_cast<int>(width), p.key_dim = static_cast<int>(key_dim);
  p.qkv_offset = conv.sc[3];
  p.q_exp = fbuf(rq, 1), p.k_exp = fbuf(rk, 1);
  p.k_heads = static_cast<int>(k_heads), p.cols = static_cast<int>(cols), p.factor = static_cast<int>(factor);
  p.eps_q = float_of_bits(lq.sc[2]), p.scale_q = float_of_bits(lq.sc[3]);
  p.eps_k = float_of_bits(lk.sc[2]), p.scale_k = float_of_bits(lk.sc[3]);
  *rc = launch_linear_mixer_inputs(p, ctx->stream);
  return *rc == kUnsupportedFeature ? 0 : 6;
}

// rmsnorm(q heads), rmsnorm(k heads), mrope(q), mrope(k) [, copy_d2d(k row -> cache), copy_d2d(v row -> cache)]
// (src/models/qwen3_5/trunk.cpp:374-391 of the reference; the copies are AppendKvRows of an fp32 cache)
size_t merged_head_norm_rope(tsr_context* ctx, const std::vector<PendingLaunch>& q, size_t i, int* rc) {
  if (!ctx->fold_elementwise || !fuse_elementwise() || i + 4 > q.size()) return 0;
  const PendingLaunch &nq = q[i], &nk = q[i + 1], &mq = q[i + 2], &mk = q[i + 3];
  if (!is_named(nq, "rmsnorm") || !is_named(nk, "rmsnorm") || !is_named(mq, "mrope") || !is_named(mk, "mrope")) return 0;
  const uint64_t heads = nq.sc[0], kv_heads = nk.sc[0], d = nq.sc[1];
  if (nk.sc[1] != d || d % 32 != 0 || d > 1024 || nq.buf[2] != nq.buf[0] || nk.buf[2] != nk.buf[0]) return 0;
  if (mq.buf[0] != nq.buf[0] || mk.buf[0] != nk.buf[0] || mq.buf[1] != mk.buf[1] || mq.sc[0] != 1 || mk.sc[0] != 1 ||
      mq.sc[1] != heads || mk.sc[1] != kv_heads || mq.sc[2] != d || mk.sc[2] != d)
    return 0;
  for (int sidx = 3; sidx < 8; ++sidx)
    if (mq.sc[sidx] != mk.sc[sidx]) return 0;
  if (overlaps(nq.buf[0], heads * d * 4, nk.buf[0], kv_heads * d * 4)) return 0;
  HeadNormRope p{};
  p.q = fbuf(nq, 0), p.k = fbuf(nk, 0), p.q_w = fbuf(nq, 1), p.k_w = fbuf(nk, 1);
  p.pos = static_cast<const unsigned long long*>(mq.buf[1]);
  p.heads = static_cast<int>(heads), p.kv_heads = static_cast<int>(kv_heads), p.head_dim = static_cast<int>(d);
  p.rope_dim = static_cast<int>(mq.sc[3]), p.theta = float_of_bits(mq.sc[4]);
  p.sec_t = static_cast<int>(mq.sc[5]), p.sec_h = static_cast<int>(mq.sc[6]);
  p.eps_q = float_of_bits(nq.sc[2]), p.eps_k = float_of_bits(nk.sc[2]);
  size_t used = 4;
  if (i + 6 <= q.size() && is_named(q[i + 4], "copy_d2d") && is_named(q[i + 5], "copy_d2d")) {
    const PendingLaunch &ck = q[i + 4], &cv = q[i + 5];
    const uint64_t row_bytes = kv_heads * d * 4;
    const unsigned char* kdst = static_cast<const unsigned char*>(ck.buf[1]) + ck.sc[1];
    const unsigned char* vdst = static_cast<const unsigned char*>(cv.buf[1]) + cv.sc[1];
    const unsigned char* vsrc = static_cast<const unsigned char*>(cv.buf[0]) + cv.sc[0];
    if (ck.buf[0] == nk.buf[0] && ck.sc[0] == 0 && ck.sc[2] == row_bytes && cv.sc[2] == row_bytes &&
        reinterpret_cast<uintptr_t>(kdst) % 4 == 0 && reinterpret_cast<uintptr_t>(vdst) % 4 == 0 &&
        reinterpret_cast<uintptr_t>(vsrc) % 4 == 0 && !overlaps(kdst, row_bytes, nq.buf[0], heads * d * 4) &&
        !overlaps(kdst, row_bytes, nk.buf[0], row_bytes) && !overlaps(vdst, row_bytes, nq.buf[0], heads * d * 4) &&
        !overlaps(vdst, row_bytes, nk.buf[0], row_bytes) && !overlaps(vdst, row_bytes, vsrc, row_bytes) &&
        !overlaps(kdst, row_bytes, vsrc, row_bytes) && !overlaps(kdst, row_bytes, vdst, row_bytes)) {
      p.k_row = reinterpret_cast<float*>(const_cast<unsigned char*>(kdst));
      p.v_src = reinterpret_cast<const float*>(vsrc);
      p.v_row = reinterpret_cast<float*>(const_cast<unsigned char*>(vdst));
      used = 6;
    }
  }
  *rc = launch_head_norm_rope(p, ctx->stream);
  return *rc == kUnsupportedFeature ? 0 : used;
}

// attention (any cache format), sigmoid_gate of its output in place (src/models/qwen3_5/trunk.cpp:441-452)
size_t merged_attention_gate(tsr_context* ctx, const std::vector<PendingLaunch>& q, size_t i, int* rc) {
  if (!ctx->fold_elementwise || !fuse_elementwise() || i + 2 > q.size() || !is_named(q[i + 1], "sigmoid_gate")) return 0;
  const PendingLaunch &at = q[i], &sg = q[i + 1];
  int fmt;
  const bool plain = is_named(at, "attention");
  if (plain) fmt = at.sc[8] != 0 ? TSR_KV_F16 : TSR_KV_F32;
  else if (is_named(at, "attention_q8")) fmt = TSR_KV_INT8;
  else if (is_named(at, "attention_q4")) fmt = TSR_KV_INT4;
  else if (is_named(at, "attention_fp8")) fmt = TSR_KV_FP8;
  else return 0;
  const int out_at = plain ? 3 : 5;
  const uint64_t m = at.sc[0], heads = at.sc[2], d = at.sc[4], row_base = at.sc[6];
  if (row_base != 0 || sg.sc[0] != m * heads * d || sg.buf[0] != at.buf[out_at] || sg.buf[2] != at.buf[out_at]) return 0;
  if (overlaps(sg.buf[1], sg.sc[0] * 4, at.buf[out_at], sg.sc[0] * 4)) return 0;
  *rc = attention_gated(fmt, fbuf(at, 0), at.buf[1], at.buf[2], plain ? nullptr : fbuf(at, 3), plain ? nullptr : fbuf(at, 4),
                        fbuf(at, out_at), fbuf(sg, 1), m, at.sc[1], heads, at.sc[3], d, at.sc[5], 0, at.sc[7], plain ? at.sc[9] : 1,
                        ctx->stream);
  return *rc == kUnsupportedFeature ? 0 : 2;
}

int issue_one(tsr_context* ctx, const PendingLaunch& op) {
  const Args a{op.buf, op.bytes, op.nbuf, op.sc, op.nsc, op.grid_y, ctx->stream, false, ctx};
  return kTable[op.kernel].fn(a);
}

// Issues the queue `q` on the context's stream, rewritten as described above.
int issue_queue(tsr_context* ctx, const std::vector<PendingLaunch>& q) {
  size_t i = 0;
  while (i < q.size()) {
    Prologue pro{};
    const float* pro_in = nullptr;
    uint64_t pro_rows = 0, pro_cols = 0;
    const bool has_pro = as_prologue(ctx, q, i, &pro, &pro_in, &pro_rows, &pro_cols);
    const size_t start = has_pro ? i + 1 : i;
    Projection first;
    if (!as_projection(q, start, &first)) {
      int rc = kOk;
      size_t merged = merged_linear_mixer_inputs(ctx, q, i, &rc);
      if (merged == 0) merged = merged_head_norm_rope(ctx, q, i, &rc);
      if (merged == 0) merged = merged_attention_gate(ctx, q, i, &rc);
      if (merged != 0) {
        if (rc != kOk) return rc;
        i += merged;
        continue;
      }
      if (int rc1 = issue_one(ctx, q[i])) return rc1;
      ++i;
      continue;
    }
    GroupTarget t[kMaxGroup];
    int count = 0;
    size_t end = start;
    const size_t a_bytes = first.m * first.k * 4;
    if (first.with_tp) {
      t[count++] = first.t;
      end += first.ops;
    }
    if (has_pro && (overlaps(first.t.c, first.m * first.t.n * 4, pro_in, a_bytes) ||
                    overlaps(first.t.c, first.m * first.t.n * 4, pro.other, a_bytes))) {
      // the projection overwrites what the folded step reads: keep the steps apart
      if (int rc = issue_one(ctx, q[i])) return rc;
      ++i;
      continue;
    }
    while (!first.with_tp && count < kMaxGroup && end < q.size()) {
      Projection next;
      if (!as_projection(q, end, &next)) break;
      if (next.with_tp || next.fmt != first.fmt || next.a != first.a || next.m != first.m || next.k != first.k) break;
      // an output that lands in the shared activations (or in what they are made from) would
      // change what later members read
      const size_t c_bytes = next.m * next.t.n * 4;
      if (overlaps(next.t.c, c_bytes, first.a, a_bytes) ||
          (has_pro && (overlaps(next.t.c, c_bytes, pro_in, a_bytes) || overlaps(next.t.c, c_bytes, pro.other, a_bytes)))) {
        if (count == 0) {
          t[count++] = next.t;
          end += next.ops;
        }
        break;
      }
      t[count++] = next.t;
      end += next.ops;
    }
    if (count == 1 && first.m <= kStagedRows) {
      Projection only = first;
      only.t = t[0];
      if (as_epilogue_add(ctx, q, end, only, has_pro ? pro_in : first.a, a_bytes, has_pro ? &pro : nullptr, &t[0])) ++end;
    }
    // with a prologue the launch reads the prologue's input; the projections' A is its output
    const float* act = has_pro ? pro_in : first.a;
    int rc = kOk;
    if (first.m <= kStagedRows) {
      rc = fused_group(ctx, first.fmt, act, t, count, first.m, first.k, first.with_tp, ctx->stream, has_pro ? &pro : nullptr);
    } else {
      // nine to sixteen rows: the merged launch twice, eight rows and the rest
      for (uint64_t i0 = 0; i0 < first.m && rc == kOk; i0 += kStagedRows) {
        GroupTarget part[kMaxGroup];
        for (int j = 0; j < count; ++j) {
          part[j] = t[j];
          part[j].c = t[j].c + i0 * t[j].n;
        }
        const uint64_t rows = first.m - i0 < kStagedRows ? first.m - i0 : kStagedRows;
        rc = fused_group(ctx, first.fmt, act + i0 * first.k, part, count, rows, first.k, false, ctx->stream, nullptr);
      }
    }
    if (rc == kUnsupportedFeature) {
      for (size_t j = i; j < end; ++j)
        if (int r = issue_one(ctx, q[j])) return r;
    } else if (rc != kOk) {
      return rc;
    }
    i = end;
  }
  return kOk;
}

uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  h *= 0xFF51AFD7ED558CCDull;
  return h ^ (h >> 29);
}

uint64_t queue_hash(const tsr_context* ctx, const std::vector<PendingLaunch>& q) {
  uint64_t h = mix(0x243F6A8885A308D3ull, reinterpret_cast<uintptr_t>(ctx->tp) ^ (ctx->fold_elementwise ? 1u : 0u));
  for (const PendingLaunch& op : q) {
    h = mix(h, (static_cast<uint64_t>(op.kernel) << 40) ^ (static_cast<uint64_t>(op.grid_y) << 8) ^
                   (static_cast<uint64_t>(op.nbuf) << 4) ^ static_cast<uint64_t>(op.nsc));
    for (int i = 0; i < op.nbuf; ++i) h = mix(h, reinterpret_cast<uintptr_t>(op.buf[i]));
    for (int i = 0; i < op.nsc; ++i) h = mix(h, op.sc[i]);
  }
  return h;
}

constexpr size_t kMaxGraphs = 32;
constexpr size_t kMinGraphOps = 8;  // shorter queues are cheaper to issue than to look up

}  // namespace

namespace tsr {

int flush_pending(tsr_context* ctx) {
  if (ctx->pending.empty()) return kOk;
  std::vector<PendingLaunch> q;
  q.swap(ctx->pending);
  ++ctx->stats.flushes;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &capturing) != cudaSuccess) {
    cudaGetLastError();
    capturing = cudaStreamCaptureStatusNone;
  }
  const bool graphs = ctx->use_graphs && capturing == cudaStreamCaptureStatusNone && q.size() >= kMinGraphOps;
  uint64_t hash = 0;
  if (graphs) {
    hash = queue_hash(ctx, q);
    auto it = ctx->graphs.find(hash);
    if (it != ctx->graphs.end() && it->second.ops == q.size()) {
      it->second.last_use = ++ctx->use_clock;
      const cudaError_t e = cudaGraphLaunch(it->second.exec, ctx->stream);
      if (e != cudaSuccess) return ctx->fail(e, "cudaGraphLaunch");
      ctx->stats.device_kernels += it->second.kernels;
      ++ctx->stats.graph_launches;
      return kOk;
    }
    if (ctx->seen_queues[hash]++ >= 1) {
      // second appearance: capture the rewritten queue, keep it, replay it
      const uint64_t before = launch_counter().load();
      if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int rc = issue_queue(ctx, q);
        cudaGraph_t graph = nullptr;
        const cudaError_t ec = cudaStreamEndCapture(ctx->stream, &graph);
        cudaGraphExec_t exec = nullptr;
        if (rc == kOk && ec == cudaSuccess && graph != nullptr &&
            cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
          cudaGraphDestroy(graph);
          if (ctx->graphs.size() >= kMaxGraphs) {
            auto oldest = ctx->graphs.begin();
            for (auto g = ctx->graphs.begin(); g != ctx->graphs.end(); ++g)
              if (g->second.last_use < oldest->second.last_use) oldest = g;
            // the stream may still be running it
            cudaStreamSynchronize(ctx->stream);
            cudaGraphExecDestroy(oldest->second.exec);
            ctx->graphs.erase(oldest);
          }
          CachedGraph cg;
          cg.exec = exec;
          cg.last_use = ++ctx->use_clock;
          cg.kernels = launch_counter().load() - before;
          cg.ops = q.size();
          ctx->graphs[hash] = cg;
          ctx->seen_queues.erase(hash);
          const cudaError_t e = cudaGraphLaunch(exec, ctx->stream);
          if (e != cudaSuccess) return ctx->fail(e, "cudaGraphLaunch");
          ctx->stats.device_kernels += cg.kernels;
          ++ctx->stats.graph_launches;
          return kOk;
        }
        if (graph != nullptr) cudaGraphDestroy(graph);
        cudaGetLastError();  // nothing ran during the failed capture: issue the queue directly below
      } else {
        cudaGetLastError();
      }
    }
    if (ctx->seen_queues.size() > 4096) ctx->seen_queues.clear();
  }
  const uint64_t before = launch_counter().load();
  const int rc = issue_queue(ctx, q);
  ctx->stats.device_kernels += launch_counter().load() - before;
  if (rc != kOk) ctx->error = "a deferred launch failed when the queue was issued";
  return rc;
}

}  // namespace tsr

namespace tsr {
// A device-to-device copy of at most kQueuedCopyLimit bytes joins the deferred queue as a "copy_d2d" launch.
int queue_copy(tsr_context* ctx, const void* src, size_t src_offset, void* dst, size_t dst_offset, size_t bytes) {
  static const int id = tsr_kernel_lookup("copy_d2d");
  PendingLaunch op{};
  op.kernel = id;
  op.grid_y = 1;
  op.nbuf = 2;
  op.nsc = 3;
  op.buf[0] = src, op.buf[1] = dst;
  op.bytes[0] = src_offset + bytes, op.bytes[1] = dst_offset + bytes;
  op.sc[0] = src_offset, op.sc[1] = dst_offset, op.sc[2] = bytes;
  ctx->pending.push_back(op);
  return kOk;
}
}  // namespace tsr

extern "C" {

int tsr_kernel_count(void) { return kCount; }

const char* tsr_kernel_name(int kernel) {
  return kernel >= 0 && kernel < kCount ? kTable[kernel].name : nullptr;
}

int tsr_kernel_lookup(const char* name) {
  if (!name) return -1;
  for (int i = 0; i < kCount; ++i)
    if (std::strcmp(kTable[i].name, name) == 0) return i;
  return -1;
}

int tsr_launch(tsr_context* ctx, int kernel, const uint32_t grid[3], const uint32_t block[3],
               const void* const* buffers, const size_t* buffer_bytes, int n_buffers,
               const uint64_t* scalars, int n_scalars) {
  if (!ctx || kernel < 0 || kernel >= kCount) return kInvalidArgument;
  // ValidateLaunch, include/tessera/backend.hpp:138-148.
  if (n_buffers < 0 || n_buffers > kMaxLaunchBuffers || n_scalars < 0 || n_scalars > kMaxLaunchScalars)
    return kInvalidArgument;
  if ((n_buffers && (!buffers || !buffer_bytes)) || (n_scalars && !scalars)) return kInvalidArgument;
  uint32_t grid_y = 0;
  if (grid) {
    if (grid[0] == 0 || grid[1] == 0 || grid[2] == 0) return kInvalidArgument;
    grid_y = grid[1];
  }
  if (block && (block[0] == 0 || block[1] == 0 || block[2] == 0)) return kInvalidArgument;
  for (int i = 0; i < n_buffers; ++i)
    if (!buffers[i]) return kInvalidArgument;
  if (int rc = ctx->select()) return rc;
  Args a{buffers, buffer_bytes, n_buffers, scalars, n_scalars, grid_y, ctx->stream, ctx->deferred, ctx};
  if (!ctx->deferred) {
    const uint64_t before = launch_counter().load();
    const int rc = kTable[kernel].fn(a);
    ctx->stats.device_kernels += launch_counter().load() - before;
    if (rc == kOk) ++ctx->stats.api_launches;
    return rc;
  }
  // deferred: the arguments are checked now, the launch is made when the queue is flushed
  if (int rc = kTable[kernel].fn(a)) return rc;
  PendingLaunch op{};
  op.kernel = kernel;
  op.grid_y = grid_y;
  op.nbuf = n_buffers;
  op.nsc = n_scalars;
  for (int i = 0; i < n_buffers; ++i) {
    op.buf[i] = buffers[i];
    op.bytes[i] = buffer_bytes[i];
  }
  for (int i = 0; i < n_scalars; ++i) op.sc[i] = scalars[i];
  ctx->pending.push_back(op);
  ++ctx->stats.api_launches;
  return kOk;
}

int tsr_launch_many(tsr_context* ctx, const tsr_launch_desc* launches, size_t count, size_t* done) {
  if (done) *done = 0;
  if (!ctx || (!launches && count)) return kInvalidArgument;
  for (size_t i = 0; i < count; ++i) {
    const tsr_launch_desc& d = launches[i];
    const int rc = tsr_launch(ctx, d.kernel, d.grid, d.block, d.buffers, d.buffer_bytes, d.n_buffers, d.scalars,
                              d.n_scalars);
    if (rc != kOk) return rc;
    if (done) *done = i + 1;
  }
  return kOk;
}

int tsr_gemv_group(tsr_context* ctx, int fmt, const float* a, const void* const* w, float* const* c,
                   const uint64_t* n, int count, uint64_t m, uint64_t k) {
  if (!ctx || !a || !w || !c || !n || count < 1 || count > kMaxGroup || (fmt != 0 && fmt != 1) || !fits_int(m) ||
      !fits_int(k) || k % 256 != 0 || !aligned16(a))
    return kInvalidArgument;
  GroupTarget t[kMaxGroup];
  for (int i = 0; i < count; ++i) {
    if (!w[i] || !c[i] || !fits_int(n[i]) || !aligned16(c[i]) || !aligned16(w[i])) return kInvalidArgument;
    t[i] = GroupTarget{w[i], c[i], n[i]};
  }
  if (int rc = ctx->select()) return rc;
  if (int rc = flush_pending(ctx)) return rc;
  int rc = fused_group(ctx, fmt, a, t, count, m, k, false, ctx->stream);
  if (rc == kUnsupportedFeature) {
    for (int i = 0; i < count; ++i) {
      rc = fmt == 0 ? tsr_gemm_q4k(a, w[i], c[i], m, n[i], k, 1, ctx->stream)
                    : tsr_gemm_q6k(a, w[i], c[i], m, n[i], k, 1, ctx->stream);
      if (rc != kOk) return rc;
    }
  }
  return rc;
}

}  // extern "C"
