"""The load-time tensor-parallel slicer (tsr_slice_shape / tsr_slice_tensor) against the
reference's SliceTensor2D built from its own sources, and the properties that hold where
the reference refuses the split.  Host memory only: runs without a GPU."""
import numpy as np
import pytest

from tessera_b200 import capi, synth
from tessera_b200.tp import (COLUMN, FMT_FP8, FMT_MXFP4, FMT_Q4K, FMT_Q6K, REPLICATED, ROW, slice_shape,
                             slice_tensor)

# the reference's DType values (include/tessera/types.hpp:93-102)
REF_DTYPE = {FMT_Q4K: 10, FMT_Q6K: 12, FMT_MXFP4: 6, FMT_FP8: 3}


def make(fmt, n, k, seed):
    if fmt == FMT_Q4K:
        return synth.q4k_weights(n, k, seed=seed)
    if fmt == FMT_Q6K:
        return synth.q6k_weights(n, k, seed=seed)
    if fmt == FMT_MXFP4:
        return synth.mxfp4_weights(n, k, seed=seed)
    return synth.fp8_weights(n, k, seed=seed)[0]


@pytest.mark.parametrize("fmt", [FMT_Q4K, FMT_Q6K, FMT_FP8])
@pytest.mark.parametrize("kind", [REPLICATED, COLUMN, ROW])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_slices_equal_the_reference_where_it_accepts_the_split(reference_oracle, fmt, kind, world):
    n, k = 24, 2048
    w = make(fmt, n, k, seed=5)
    for rank in range(world):
        want = reference_oracle.slice_tensor2d(REF_DTYPE[fmt], n, k, kind, rank, world, w)
        assert not isinstance(want, int), want
        ref_bytes, ref_rows, ref_cols = want
        rows, cols, _, nbytes = slice_shape(fmt, kind, n, k, rank, world)
        assert (rows, cols, nbytes) == (ref_rows, ref_cols, ref_bytes.size)
        assert np.array_equal(slice_tensor(fmt, kind, n, k, rank, world, w), ref_bytes)


@pytest.mark.parametrize("world", [2, 4])
def test_mxfp4_column_slices_equal_the_reference(reference_oracle, world):
    n, k = 24, 1024
    w = make(FMT_MXFP4, n, k, seed=6)
    for rank in range(world):
        ref_bytes, ref_rows, ref_cols = reference_oracle.slice_tensor2d(REF_DTYPE[FMT_MXFP4], n, k, COLUMN, rank, world, w)
        assert np.array_equal(slice_tensor(FMT_MXFP4, COLUMN, n, k, rank, world, w), ref_bytes)
        assert slice_shape(FMT_MXFP4, COLUMN, n, k, rank, world)[:2] == (ref_rows, ref_cols)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_mxfp4_row_slices_keep_the_kernel_layout(reference_oracle, world):
    """The reference's row-kind MXFP4 output interleaves each row's scales with its nibbles; the
    kernels read all nibbles, then all scales.  Same bytes per row, the layout of the kernels."""
    n, k = 8, 2048
    w = make(FMT_MXFP4, n, k, seed=7)
    blob, scales = w[: n * k // 2].reshape(n, k // 2), w[n * k // 2:].reshape(n, k // 32)
    for rank in range(world):
        rows, cols, c0, nbytes = slice_shape(FMT_MXFP4, ROW, n, k, rank, world)
        got = slice_tensor(FMT_MXFP4, ROW, n, k, rank, world, w)
        assert got.size == nbytes == n * cols // 2 + n * cols // 32
        assert np.array_equal(got[: n * cols // 2].reshape(n, -1), blob[:, c0 // 2:(c0 + cols) // 2])
        assert np.array_equal(got[n * cols // 2:].reshape(n, -1), scales[:, c0 // 32:(c0 + cols) // 32])
        ref = reference_oracle.slice_tensor2d(REF_DTYPE[FMT_MXFP4], n, k, ROW, rank, world, w)
        ref_rows = ref[0].reshape(n, -1)  # per row: nibbles, then scales
        assert np.array_equal(ref_rows[:, : cols // 2], got[: n * cols // 2].reshape(n, -1))
        assert np.array_equal(ref_rows[:, cols // 2:], got[n * cols // 2:].reshape(n, -1))


@pytest.mark.parametrize("fmt,block", [(FMT_Q4K, 144), (FMT_Q6K, 210)])
def test_uneven_row_split_is_accepted_and_covers_every_block(reference_oracle, fmt, block):
    """K = 17408 on 8 ranks is 8.5 blocks per rank: the reference refuses it
    (tensor_slice.cpp:145-147); the slicer hands out ranges of 8 and 9 whole blocks."""
    n, k, world = 4, 17408, 8
    w = make(fmt, n, k, seed=8)
    assert reference_oracle.slice_tensor2d(REF_DTYPE[fmt], n, k, ROW, 1, world, w) == -int(capi.StatusCode.InvalidArgument)
    full = w.reshape(n, k // 256, block)
    pieces, begin = [], 0
    for rank in range(world):
        rows, cols, c0, nbytes = slice_shape(fmt, ROW, n, k, rank, world)
        assert rows == n and c0 == begin and cols % 256 == 0 and cols // 256 in (8, 9)
        part = slice_tensor(fmt, ROW, n, k, rank, world, w).reshape(n, cols // 256, block)
        assert np.array_equal(part, full[:, c0 // 256:(c0 + cols) // 256])
        pieces.append(part)
        begin += cols
    assert begin == k
    assert np.array_equal(np.concatenate(pieces, axis=1), full)


def test_bad_arguments_are_refused():
    lib = capi.load_library()
    w = make(FMT_Q4K, 4, 512, seed=9)
    with pytest.raises(capi.StatusError):
        slice_shape(FMT_Q4K, ROW, 4, 500, 0, 2)        # not whole blocks
    with pytest.raises(capi.StatusError):
        slice_shape(FMT_Q4K, ROW, 4, 512, 2, 2)        # rank out of range
    with pytest.raises(capi.StatusError):
        slice_shape(FMT_Q4K, ROW, 4, 512, 0, 4)        # fewer blocks than ranks: an empty shard
    with pytest.raises(capi.StatusError):
        slice_shape(7, ROW, 4, 512, 0, 2)              # unknown format
    dst = np.empty(16, dtype=np.uint8)                 # destination too small
    assert lib.tsr_slice_tensor(FMT_Q4K, COLUMN, 4, 512, 0, 2, w.ctypes.data, w.nbytes, dst.ctypes.data,
                                dst.nbytes) == capi.StatusCode.InvalidArgument
    assert lib.tsr_slice_tensor(FMT_Q4K, COLUMN, 4, 512, 0, 2, w.ctypes.data, 100, dst.ctypes.data,
                                dst.nbytes) == capi.StatusCode.InvalidArgument


def test_explicit_ranges_cut_the_same_bytes():
    from tessera_b200.tp import slice_range
    n, k = 12, 17408
    w = make(FMT_Q6K, n, k, seed=10)
    full = w.reshape(n, k // 256, 210)
    # a Q6_K row split in units of four blocks: every rank's rows stay 8-byte aligned
    got = slice_range(FMT_Q6K, n, k, 0, n, 56 * 256, 68 * 256, w).reshape(n, 12, 210)
    assert np.array_equal(got, full[:, 56:68])
    # a column split that follows an uneven k range of the projection it feeds
    got = slice_range(FMT_Q6K, n, k, 3, 10, 0, k, w).reshape(7, k // 256, 210)
    assert np.array_equal(got, full[3:10])
    wm = make(FMT_MXFP4, n, 1024, seed=11)
    got = slice_range(FMT_MXFP4, n, 1024, 2, 6, 256, 768, wm)
    blob, sc = wm[: n * 512].reshape(n, 512), wm[n * 512:].reshape(n, 32)
    assert np.array_equal(got[: 4 * 256].reshape(4, 256), blob[2:6, 128:384])
    assert np.array_equal(got[4 * 256:].reshape(4, 16), sc[2:6, 8:24])
    with pytest.raises(capi.StatusError):
        slice_range(FMT_Q6K, n, k, 0, n, 100, 356, w)   # not on block boundaries
