// Tensor-parallel weight slicing at load time (host memory to host memory).
//
// Mirrors the reference's SliceTensor2D / SliceMxFp4
// (src/core/loaders/tensor_slice.cpp:50-159) for the four weight formats of the
// projection path, with one extension: a row-parallel (K) split may be uneven.
// The reference computes the column range as cols*rank/world and rejects it
// when it does not fall on a block boundary (tensor_slice.cpp:145-147), which
// refuses K = 17408 on 8 ranks (8.5 Q4_K blocks each).  Here the same floor
// formula is applied to the block count, so rank r keeps blocks
// [nblocks*r/world, nblocks*(r+1)/world): the same ranges whenever the
// reference accepts the split, ranges that differ by one block otherwise.
// The caller slices the activations of a row-parallel projection with the same
// range (tsr_slice_shape reports it).
//
// Layouts: Q4_K / Q6_K rows of k/256 blocks of 144 / 210 bytes; FP8 rows of k
// bytes (the fp32 row scales are sliced by the caller: a row range for a column
// split, all of them for a row split); MXFP4 n*k/2 nibble bytes followed by
// n*k/32 E8M0 bytes, kept in that layout in the output (the reference's
// row-kind MXFP4 output interleaves each row's scales with its nibbles,
// tensor_slice.cpp:93-98, a layout none of its kernels read; only its GGUF
// path is ever sliced, src/core/loaders/mxfp4.cpp:180-184).
#include <cstdint>
#include <cstring>

#include "launch.h"
#include "tessera_b200.h"

namespace {

struct Unit {
  uint64_t elements, bytes;  // one indivisible run of a row
};

bool unit_of(int fmt, Unit* u) {
  switch (fmt) {
    case 0: *u = {256, 144}; return true;  // Q4_K
    case 1: *u = {256, 210}; return true;  // Q6_K
    case 2: *u = {32, 16}; return true;    // MXFP4: 16 nibble bytes (+ 1 scale byte, kept apart)
    case 3: *u = {1, 1}; return true;      // FP8 E4M3
    default: return false;
  }
}

struct Range {
  uint64_t r0, r1, u0, u1;  // kept rows and kept units of every row
};

int plan(int fmt, int kind, uint64_t rows, uint64_t cols, int rank, int world, Range* out, Unit* unit) {
  if (!unit_of(fmt, unit) || rows == 0 || cols == 0 || cols % unit->elements != 0) return tsr::kInvalidArgument;
  const uint64_t units = cols / unit->elements;
  *out = {0, rows, 0, units};
  if (kind == 0 || world <= 1) return tsr::kOk;  // ParallelKind::Replicated
  if (rank < 0 || rank >= world) return tsr::kInvalidArgument;
  const uint64_t r = static_cast<uint64_t>(rank), w = static_cast<uint64_t>(world);
  if (kind == 1) {  // ParallelKind::Column: output rows
    out->r0 = rows * r / w;
    out->r1 = rows * (r + 1) / w;
    return tsr::kOk;
  }
  if (kind == 2) {  // ParallelKind::Row: input columns, whole blocks
    out->u0 = units * r / w;
    out->u1 = units * (r + 1) / w;
    return out->u1 > out->u0 ? tsr::kOk : tsr::kInvalidArgument;
  }
  return tsr::kInvalidArgument;
}

uint64_t tensor_bytes(int fmt, uint64_t rows, uint64_t units, const Unit& unit) {
  return rows * units * unit.bytes + (fmt == 2 ? rows * units : 0);
}

}  // namespace

extern "C" {

int tsr_slice_shape(int fmt, int kind, uint64_t rows, uint64_t cols, int rank, int world, uint64_t* out_rows,
                    uint64_t* out_cols, uint64_t* col_begin, uint64_t* out_bytes) {
  Range g;
  Unit unit;
  if (int rc = plan(fmt, kind, rows, cols, rank, world, &g, &unit)) return rc;
  if (out_rows) *out_rows = g.r1 - g.r0;
  if (out_cols) *out_cols = (g.u1 - g.u0) * unit.elements;
  if (col_begin) *col_begin = g.u0 * unit.elements;
  if (out_bytes) *out_bytes = tensor_bytes(fmt, g.r1 - g.r0, g.u1 - g.u0, unit);
  return tsr::kOk;
}

int tsr_slice_range(int fmt, uint64_t rows, uint64_t cols, uint64_t row_begin, uint64_t row_end, uint64_t col_begin,
                    uint64_t col_end, const void* src, size_t src_bytes, void* dst, size_t dst_bytes) {
  Unit unit;
  if (!src || !dst || !unit_of(fmt, &unit) || rows == 0 || cols == 0 || cols % unit.elements != 0 ||
      row_begin >= row_end || row_end > rows || col_begin >= col_end || col_end > cols ||
      col_begin % unit.elements != 0 || col_end % unit.elements != 0)
    return tsr::kInvalidArgument;
  const uint64_t units = cols / unit.elements, u0 = col_begin / unit.elements, u1 = col_end / unit.elements;
  const uint64_t keep_rows = row_end - row_begin, keep_units = u1 - u0;
  if (tensor_bytes(fmt, rows, units, unit) > src_bytes || tensor_bytes(fmt, keep_rows, keep_units, unit) > dst_bytes)
    return tsr::kInvalidArgument;
  const auto* s = static_cast<const unsigned char*>(src);
  auto* d = static_cast<unsigned char*>(dst);
  const uint64_t row_bytes = units * unit.bytes, kept = keep_units * unit.bytes;
  for (uint64_t r = 0; r < keep_rows; ++r)
    std::memcpy(d + r * kept, s + (row_begin + r) * row_bytes + u0 * unit.bytes, kept);
  if (fmt == 2) {
    const unsigned char* ss = s + rows * row_bytes;
    unsigned char* ds = d + keep_rows * kept;
    for (uint64_t r = 0; r < keep_rows; ++r)
      std::memcpy(ds + r * keep_units, ss + (row_begin + r) * units + u0, keep_units);
  }
  return tsr::kOk;
}

int tsr_slice_tensor(int fmt, int kind, uint64_t rows, uint64_t cols, int rank, int world, const void* src,
                     size_t src_bytes, void* dst, size_t dst_bytes) {
  Range g;
  Unit unit;
  if (int rc = plan(fmt, kind, rows, cols, rank, world, &g, &unit)) return rc;
  return tsr_slice_range(fmt, rows, cols, g.r0, g.r1, g.u0 * unit.elements, g.u1 * unit.elements, src, src_bytes, dst,
                         dst_bytes);
}

}  // extern "C"
