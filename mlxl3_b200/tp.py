"""Tensor-parallel sharding of an EXL3 linear layer (one process per GPU).

The layer's own structure gives exact shards, because both rotations act on independent 128-blocks:

* column-parallel (q/k/v, gate/up): rank r keeps output columns ``[r*out/W, (r+1)*out/W)`` -- the trellis
  tile columns, ``svh`` and ``bias`` of that range and all of ``suh``.  No communication; the ranks' outputs
  concatenate to the full output.
* row-parallel (o, down): rank r keeps input rows ``[r*in/W, (r+1)*in/W)`` -- the trellis tile rows and
  ``suh`` of that range and all of ``svh``.  Each rank produces a full-width fp32 partial sum, exactly the
  split-K partial of the reference (native/src/linear.rs:978-982); the partials are summed across ranks
  (all-reduce) and the output rotation runs on the sum (``Exl3Linear.forward_partial_device`` then
  ``finish_device``).

Shards must stay multiples of 128 in the sharded dimension.
"""
from __future__ import annotations

import numpy as np


def shard_dims(kind: str, n_in: int, n_out: int, world: int) -> tuple[int, int]:
    """(in, out) of one rank's shard; ``kind`` is "col" or "row"."""
    if kind not in ("col", "row"):
        raise ValueError(f"unknown tensor-parallel kind {kind!r}")
    if world < 1:
        raise ValueError("world size must be positive")
    if world == 1:
        return n_in, n_out
    full = n_out if kind == "col" else n_in
    if full % (128 * world):
        raise ValueError(f"{full} does not split into {world} shards of whole 128-blocks")
    return (n_in, n_out // world) if kind == "col" else (n_in // world, n_out)


def column_shard(trellis: np.ndarray, suh: np.ndarray, svh: np.ndarray, bias: np.ndarray | None, rank: int, world: int):
    """(trellis, suh, svh, bias) of rank ``rank`` for a column-parallel layer."""
    n_in, n_out = trellis.shape[0] * 16, trellis.shape[1] * 16
    _, s_out = shard_dims("col", n_in, n_out, world)
    lo, hi = rank * s_out, (rank + 1) * s_out
    return (np.ascontiguousarray(trellis[:, lo // 16:hi // 16]), suh, np.ascontiguousarray(svh[lo:hi]),
            None if bias is None else np.ascontiguousarray(bias[lo:hi]))


def row_shard(trellis: np.ndarray, suh: np.ndarray, svh: np.ndarray, bias: np.ndarray | None, rank: int, world: int):
    """(trellis, suh, svh, bias) of rank ``rank`` for a row-parallel layer, and the slice of the input it reads.
    ``svh`` and ``bias`` are whole: they apply after the sum over ranks."""
    n_in, n_out = trellis.shape[0] * 16, trellis.shape[1] * 16
    s_in, _ = shard_dims("row", n_in, n_out, world)
    lo, hi = rank * s_in, (rank + 1) * s_in
    return (np.ascontiguousarray(trellis[lo // 16:hi // 16]), np.ascontiguousarray(suh[lo:hi]), svh, bias), slice(lo, hi)
