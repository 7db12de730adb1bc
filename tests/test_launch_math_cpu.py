"""Index arithmetic of the INT4 GEMV launch, restated on the CPU.

The kernel (metile_b200/csrc/affine_gemv.cuh) hands row blocks blockIdx, blockIdx + grid, ... to a
CTA and lets it run `(row_blocks - 1 - blockIdx) / grid + 1` passes, in unsigned arithmetic.  That
is only right while the grid has at most `row_blocks` CTAs, which the launcher guarantees by
construction; these checks pin both halves for the shapes the library is used with."""

import pytest

SM_COUNT = 148
WARPS = 8


def ksplit_of(k, n):
    ksplit, slots = 1, k >> 5
    while ksplit < 8 and n * ksplit < 16384 and slots // (ksplit * 2) >= 16:
        ksplit *= 2
    return ksplit


def rows_per_half_warp(rows, dual):
    if dual:
        return 2 if rows <= 2 else 1
    return 4 if rows <= 2 else (2 if rows <= 4 else 1)


def launch_geometry(rows, dual, k, n, staged_bytes):
    ksplit = ksplit_of(k, n)
    rows_per_cta = (WARPS // ksplit) * 2 * rows_per_half_warp(rows, dual)
    row_blocks = -(-n // rows_per_cta)
    cap = SM_COUNT * (3 if rows == 1 and staged_bytes <= 72 * 1024 else 2)
    return rows_per_cta, row_blocks, min(row_blocks, cap)


SHAPES = [(1536, 8960), (8960, 1536), (2048, 8192), (8192, 2048), (2048, 128256), (5120, 27648),
          (27648, 5120), (5120, 3456), (3456, 5120), (1536, 256), (64, 64), (4096, 1000)]


@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("rows", [1, 2, 4, 8])
@pytest.mark.parametrize("dual", [False, True])
def test_every_row_block_runs_exactly_once(k, n, rows, dual):
    staged = k * 4 + (k >> 5) * 4 if rows == 1 else rows * k * 2
    rows_per_cta, row_blocks, grid = launch_geometry(rows, dual, k, n, staged)
    assert 1 <= grid <= row_blocks
    seen = [0] * row_blocks
    for cta in range(grid):
        passes = ((row_blocks - 1 - cta) & 0xFFFFFFFF) // grid + 1
        assert passes >= 1
        for p in range(passes):
            block = p * grid + cta
            assert block < row_blocks  # a pass never starts at or beyond the last row
            seen[block] += 1
    assert seen == [1] * row_blocks
    assert (row_blocks - 1) * rows_per_cta < n <= row_blocks * rows_per_cta


def test_pass_counts_differ_by_at_most_one():
    # N = 8192 with 16-row CTAs: 512 row blocks over 444 CTAs -- 68 CTAs run two passes, the rest one
    # (every CTA used to run two, most of them on rows past the end).
    rows_per_cta, row_blocks, grid = launch_geometry(1, True, 2048, 8192, 2048 * 4 + 256)
    assert (rows_per_cta, row_blocks, grid) == (16, 512, 444)
    passes = [(row_blocks - 1 - cta) // grid + 1 for cta in range(grid)]
    assert passes.count(2) == 68 and passes.count(1) == 376
