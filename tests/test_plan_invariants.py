"""The launch planners' invariants over an exhaustive small domain (no GPU needed: b200exl3_plan_query is host
arithmetic).  The reference proves the corresponding properties of its own split policy with Kani
(native/src/contracts.rs:1995-2012, 1051-1069); here every shape of the domain is simply checked.

Invariants:
* fused kernel and decode-step kernel (warp-level stream-K, a layer dealt out in whole rows of 8 tiles): a warp's range
  never exceeds one 128-column block's worth (so it touches at most two blocks and owns two staging buffers), the
  stated bound on the CTAs that share a column block holds for every block, every tile belongs to exactly one warp;
  where every block goes to a whole number of warps, no warp works on two blocks and the largest share did not grow;
* tensor-core product: every input split keeps at least 8 stages of 64 inputs (or there is one split), the token
  tiles cover the rows, the small shape is used up to 64 rows.
"""
import ctypes

import numpy as np
import pytest

from mlxl3_b200 import _lib


def query(kind, n_in, n_out, k, rows):
    out = (ctypes.c_int64 * 8)()
    _lib.call("b200exl3_plan_query", kind.encode(), n_in, n_out, k, rows, out, 8)
    return list(out)


def partition_ok(tiles_k, col_blocks, warps, warps_per_cta, max_pieces, whole_rows=False, whole_warps_per_block=False):
    ub = tiles_k * 8
    total = ub * col_blocks
    if whole_warps_per_block:      # block c gets warps [c W / C, (c + 1) W / C), which share its rows evenly
        w = np.arange(warps, dtype=np.int64)
        c = ((w + 1) * col_blocks - 1) // warps
        first, count = c * warps // col_blocks, (c + 1) * warps // col_blocks - c * warps // col_blocks
        assert (count >= 1).all()
        begin = np.append(8 * (c * tiles_k + tiles_k * (w - first) // count), total)
        some = begin[1:] > begin[:-1]
        assert (begin[:-1][some] // ub == (begin[1:][some] - 1) // ub).all()                 # no warp works on two blocks
        assert np.diff(begin).max() <= 8 * -(-(tiles_k * col_blocks) // warps)              # and the largest share did not grow
    elif whole_rows:      # the decode-step kernel deals a layer out in rows of 8 tiles
        begin = 8 * ((np.arange(warps + 1, dtype=np.int64) * (total // 8)) // warps)
    else:
        begin = np.minimum((np.arange(warps + 1, dtype=np.int64) * total) // warps, total)
    assert begin[0] == 0 and begin[-1] == total and (np.diff(begin) >= 0).all()          # every tile once
    assert np.diff(begin).max() <= ub                                                     # at most two blocks per warp
    ctas = warps // warps_per_cta
    cta_begin = begin[::warps_per_cta]
    first_block, last_block = cta_begin[:-1] // ub, (np.maximum(cta_begin[1:], cta_begin[:-1] + 1) - 1) // ub
    has = cta_begin[1:] > cta_begin[:-1]
    per_block = np.zeros(col_blocks + 1, np.int64)
    for c in range(ctas):
        if has[c]:
            per_block[first_block[c]:last_block[c] + 1] += 1
    assert per_block.max() <= max_pieces, (per_block.max(), max_pieces)
    return True


DIMS_IN = [128, 256, 512, 1024, 2048, 4096, 14336]
DIMS_OUT = [128, 256, 384, 1024, 4096, 6144, 14336, 28672]


@pytest.mark.parametrize("k", [1, 4, 8])
def test_fused_kernel_partition(k):
    for n_in in DIMS_IN:
        for n_out in DIMS_OUT:
            for rows in (1, 2, 3, 8, 9, 16):
                grid, max_pieces, col_blocks, warps_per_cta, smem, fused = query("qmv", n_in, n_out, k, rows)[:6]
                assert col_blocks == n_out // 128 and grid >= 1 and smem <= 200 * 1024
                assert fused == (1 if rows <= 2 else 0)
                # the kernel derives the way a layer is dealt out from the launch itself: whole warps per column block
                # when that does not raise the largest share of rows
                warps, rb = grid * warps_per_cta, n_in // 16
                per_block = warps // col_blocks
                whole = per_block >= 1 and -(-rb // per_block) <= -(-(rb * col_blocks) // warps)
                assert partition_ok(rb, col_blocks, warps, warps_per_cta, max_pieces, whole_rows=True, whole_warps_per_block=whole)


@pytest.mark.parametrize("k", [2, 4, 6])
def test_decode_step_partition(k):
    seen_modes = set()
    for n_in in DIMS_IN:
        for n_out in DIMS_OUT:
            grid, max_pieces, col_blocks, warps_per_cta, smem, warps, narrow, ok = query("stack", n_in, n_out, k, 1)
            assert ok == 1 and grid == 148 and smem <= 224 * 1024
            assert warps % warps_per_cta == 0 and 0 < warps <= grid * warps_per_cta
            assert narrow & 1 == (1 if (n_in // 16 * 8 * col_blocks + 1) * warps < 0xFFFFFFFF else 0)
            assert partition_ok(n_in // 16, col_blocks, warps, warps_per_cta, max_pieces, whole_rows=True, whole_warps_per_block=bool(narrow & 2))
            seen_modes.add(narrow & 2)
    assert seen_modes == {0, 2}                               # both ways of dealing a layer out occur in the domain
    # a layer with more column blocks than the grid has warps cannot be one pass of the step
    assert query("stack", 128, 128 * 4000, k, 1)[7] == 0


def test_tensor_core_splits():
    for n_in in DIMS_IN:
        for n_out in DIMS_OUT:
            for rows in (9, 16, 64, 65, 256, 512, 513, 2048):
                splits, token_tiles, small, stages = query("qmm", n_in, n_out, 4, rows)[:4]
                assert stages == n_in // 64 and splits >= 1
                assert splits == 1 or stages // splits >= 8
                assert small == (1 if rows <= 64 else 0)
                tile = 64 if small else 512
                assert token_tiles == -(-rows // tile)


def test_query_validation():
    lib = _lib.load()
    out = (ctypes.c_int64 * 8)()
    assert lib.b200exl3_plan_query(b"qmv", 100, 128, 4, 1, out, 8) == -1 and b"invalid plan query" in lib.b200exl3_last_error()
    assert lib.b200exl3_plan_query(b"nope", 128, 128, 4, 1, out, 8) == -1 and b"unknown plan kind" in lib.b200exl3_last_error()
    assert lib.b200exl3_plan_query(b"qmv", 128, 128, 4, 1, out, 4) == -1
