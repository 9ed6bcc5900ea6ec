// Typed projection launchers and the name-keyed kernel table.
//
// Every id below is a built-in name of the reference's kernel contract; the
// comment beside it names the reference source that defines the contract.
// One CUDA launcher can serve several ids because the contract is the result
// for the given (buffers, scalars), not the reference's thread mapping.
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "launch.h"
#include "tessera_b200.h"

using namespace tsr;

struct tsr_context;
extern "C" void* tsr_context_stream(const tsr_context* ctx);

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
template <typename Launch>
int staged_in_chunks(uint64_t m, uint64_t n, Launch launch) {
  if (m > staged_batch_max() || tile_fills_device(n)) return kUnsupportedFeature;
  for (uint64_t i0 = 0; i0 < m; i0 += kStagedRows) {
    const uint64_t rows = m - i0 < kStagedRows ? m - i0 : kStagedRows;
    const int rc = launch(i0, rows);
    if (rc != kOk) return rc;  // kUnsupportedFeature can only come from the first chunk
  }
  return kOk;
}

}  // namespace

extern "C" {

int tsr_gemm_q4k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream) {
  if (!a || !w || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) || k % 256 != 0 ||
      split == 0 || (k / 256) % split != 0 || split > 65535)
    return kInvalidArgument;
  if (!aligned16(a) || !aligned16(w) || !aligned16(c)) return kInvalidArgument;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = (m > kStagedRows && split == 1)
                     ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
                         return staged_gemm_q4k(a + i0 * k, w, c + i0 * n, rows, n, k, 1, st);
                       })
                     : staged_gemm_q4k(a, w, c, m, n, k, split, st);
  if (rc != kUnsupportedFeature) return rc;
  if (m >= 9 && split == 1) {
    const int rt = umma_gemm(0, a, w, nullptr, c, m, n, k, static_cast<cudaStream_t>(stream));
    if (rt != kUnsupportedFeature) return rt;
  }
  return rows_gemm_q4k(a, w, c, m, n, k, split, static_cast<cudaStream_t>(stream));
}

int tsr_gemm_q6k(const float* a, const void* w, float* c, uint64_t m, uint64_t n, uint64_t k,
                 uint64_t split, void* stream) {
  if (!a || !w || !c || !fits_int(m) || !fits_int(n) || !fits_int(k) || k % 256 != 0 ||
      split == 0 || (k / 256) % split != 0 || split > 65535)
    return kInvalidArgument;
  if (!aligned16(a) || (reinterpret_cast<uintptr_t>(w) & 1u) || !aligned16(c))
    return kInvalidArgument;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = (m > kStagedRows && split == 1)
                     ? staged_in_chunks(m, n, [&](uint64_t i0, uint64_t rows) {
                         return staged_gemm_q6k(a + i0 * k, w, c + i0 * n, rows, n, k, 1, st);
                       })
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
  return tsr_quantize_fp8_pack(static_cast<const float*>(a.buf[0]), const_cast<void*>(a.buf[1]),
                               static_cast<float*>(const_cast<void*>(a.buf[2])), rows, cols,
                               a.stream);
}

// round_bf16: buffer x; scalar n (backend.hpp:341-345).
int k_round(const Args& a) {
  if (!shape(a, 1, 1)) return kInvalidArgument;
  if (a.sc[0] == 0 || !holds(a, 0, a.sc[0] * 4)) return kInvalidArgument;
  return tsr_round_bf16(static_cast<float*>(const_cast<void*>(a.buf[0])), a.sc[0], a.stream);
}

// add: buffers A, B, O; scalar n (backend.hpp:258-260).
int k_add(const Args& a) {
  if (!shape(a, 3, 1)) return kInvalidArgument;
  const uint64_t n = a.sc[0];
  if (n == 0 || !holds(a, 0, n * 4) || !holds(a, 1, n * 4) || !holds(a, 2, n * 4))
    return kInvalidArgument;
  return tsr_add(static_cast<const float*>(a.buf[0]), static_cast<const float*>(a.buf[1]),
                 static_cast<float*>(const_cast<void*>(a.buf[2])), n, a.stream);
}

// fill: buffer int32; scalars value, count (backend.hpp:151-152).
int k_fill(const Args& a) {
  if (!shape(a, 1, 2)) return kInvalidArgument;
  const uint64_t n = a.sc[1];
  if (n == 0 || !holds(a, 0, n * 4)) return kInvalidArgument;
  return tsr_fill(static_cast<int32_t*>(const_cast<void*>(a.buf[0])),
                  static_cast<int32_t>(a.sc[0]), n, a.stream);
}

struct Entry {
  const char* name;
  int (*fn)(const Args&);
};

const Entry kTable[] = {
    {"fill", k_fill},
    {"add", k_add},
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
};
constexpr int kCount = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));

}  // namespace

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
  if (n_buffers < 0 || n_buffers > 16 || n_scalars < 0 || n_scalars > 16) return kInvalidArgument;
  if ((n_buffers && (!buffers || !buffer_bytes)) || (n_scalars && !scalars)) return kInvalidArgument;
  uint32_t grid_y = 0;
  if (grid) {
    if (grid[0] == 0 || grid[1] == 0 || grid[2] == 0) return kInvalidArgument;
    grid_y = grid[1];
  }
  if (block && (block[0] == 0 || block[1] == 0 || block[2] == 0)) return kInvalidArgument;
  for (int i = 0; i < n_buffers; ++i)
    if (!buffers[i]) return kInvalidArgument;
  int device = 0;
  cudaGetDevice(&device);
  extern int tsr_context_device(const tsr_context*);
  if (device != tsr_context_device(ctx)) cudaSetDevice(tsr_context_device(ctx));
  Args a{buffers, buffer_bytes, n_buffers, scalars, n_scalars, grid_y,
         static_cast<cudaStream_t>(tsr_context_stream(ctx))};
  return kTable[kernel].fn(a);
}

}  // extern "C"
