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


class TpContext:
    """Peer-memory exchange buffers of one rank (``b200exl3_tp_*``).

    ``exchange`` is a callable that takes this rank's 64-byte handle and returns the list of all ranks'
    handles in rank order (for example ``torch.distributed.all_gather_object``); the library itself has no
    communication layer.  ``finish(layer, d_yhat, rows, dtype, d_y, stream)`` then replaces the all-reduce and
    the output rotation of a row-parallel layer by one kernel launch.
    """

    def __init__(self, rank: int, world: int, max_units: int, exchange):
        import ctypes
        from ctypes import byref, c_void_p

        from . import _lib
        self.rank, self.world, self.max_units = rank, world, max_units
        own = c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.call("b200exl3_tp_alloc", world, max_units, byref(own), handle)
        self._own = own.value
        handles = exchange(handle.raw)
        if len(handles) != world or handles[rank] != handle.raw:
            raise ValueError("exchange must return every rank's handle in rank order")
        self._peers = []
        pointers = (c_void_p * world)()
        for r, raw in enumerate(handles):
            if r == rank:
                pointers[r] = self._own
                continue
            peer = c_void_p()
            _lib.call("b200exl3_tp_open", raw, byref(peer))
            self._peers.append(peer.value)
            pointers[r] = peer.value
        ctx = c_void_p()
        _lib.call("b200exl3_tp_create", rank, world, max_units, pointers, byref(ctx))
        self.handle = ctx.value

    def finish(self, layer, d_yhat: int, rows: int, dtype: int, d_y: int, stream) -> None:
        from ctypes import c_void_p

        from . import _lib
        _lib.call("b200exl3_linear_finish_tp", c_void_p(layer.handle), c_void_p(self.handle), c_void_p(d_yhat), rows, dtype,
                  c_void_p(d_y), c_void_p(stream.handle))

    def forward(self, layer, d_x: int, dtype: int, rows: int, d_y: int, workspace, stream) -> None:
        """The whole row-parallel layer in one launch (``b200exl3_linear_forward_tp``): ``d_x`` is this rank's
        slice of the input columns, ``d_y`` receives the full-width output, identical on every rank."""
        from ctypes import c_void_p

        from . import _lib
        _lib.call("b200exl3_linear_forward_tp", c_void_p(layer.handle), c_void_p(self.handle), c_void_p(d_x), dtype, rows,
                  c_void_p(d_y), c_void_p(workspace.ptr), workspace.nbytes, c_void_p(stream.handle))

    def status(self) -> int:
        from ctypes import byref, c_int, c_void_p

        from . import _lib
        out = c_int()
        _lib.call("b200exl3_tp_status", c_void_p(self.handle), byref(out))
        return out.value

    def reset(self) -> None:
        """After a wait gave up (status 4): clears this rank's inbox, use counts and status.  Every rank calls it,
        between steps, once all ranks have stopped launching."""
        from ctypes import c_void_p

        from . import _lib
        _lib.call("b200exl3_tp_reset", c_void_p(self.handle))

    def close(self) -> None:
        """Call on every rank after all ranks have finished using the buffers."""
        from ctypes import c_void_p

        from . import _lib
        if getattr(self, "handle", None):
            _lib.load().b200exl3_tp_free(c_void_p(self.handle))
            self.handle = None
            for peer in self._peers:
                _lib.load().b200exl3_tp_close(c_void_p(peer))
            self._peers = []
            _lib.load().b200exl3_free(c_void_p(self._own))
            self._own = None
