"""``Exl3Stack`` -- a decode step (a sequence of ``Exl3Linear`` / ``Exl3Group`` layers with fixed device buffers) run
as ONE persistent kernel launch (``b200exl3_stack_*``).  It plays the part of the reference's recorded decode step
(``mlxl3_replay_capture`` / ``mlxl3_replay_apply``, native/ffi/mlx_bridge.cpp:150-175): build once, replay per token.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_size_t, c_void_p

from . import _lib
from ._lib import B200Exl3Error
from .linear import Exl3Group
from .runtime import DEFAULT_STREAM, Stream


class _StackOp(ctypes.Structure):
    _fields_ = [("linear", c_void_p), ("group", c_void_p), ("d_x", c_void_p), ("d_y", c_void_p * 8), ("tp", c_void_p),
                ("fused", c_void_p)]


class Exl3Stack:
    """``Exl3Stack(ops, dtype, rows)`` with ``ops`` a list of ``(layer, d_x, d_ys)``, ``(layer, d_x, d_ys, tp_context)`` or
    ``(layer, d_x, d_ys, tp_context_or_None, prologue)``: ``layer`` an ``Exl3Linear`` or ``Exl3Group``, ``d_x`` the device
    address of its ``[rows, in]`` input, ``d_ys`` one device address (or a list, one per member of a group) for its
    outputs, ``prologue`` a ``linear.Prologue`` with the operators fused around the layer (SwiGLU or RMSNorm-from-block-sums
    in front, residual add or rotary embedding + cache append behind).  ``forward()`` runs every layer in order; layer
    i+1 may read what layer i wrote."""

    def __init__(self, ops, dtype: int, rows: int = 1):
        ops = list(ops)
        if not ops:
            raise B200Exl3Error("a step needs between 1 and 256 layers")
        table = (_StackOp * len(ops))()
        self._keep = []
        for entry, op in zip(table, ops):
            layer, d_x, d_ys = op[0], op[1], op[2]
            tp = op[3] if len(op) > 3 else None
            if isinstance(layer, Exl3Group):
                entry.group = layer.handle
            else:
                entry.linear = layer.handle
            entry.d_x = d_x
            ys = list(d_ys) if isinstance(d_ys, (list, tuple)) else [d_ys]
            if len(ys) > 8:
                raise B200Exl3Error("a layer has at most 8 outputs")
            for i, y in enumerate(ys):
                entry.d_y[i] = y
            entry.tp = tp.handle if tp is not None else None
            fused = op[4] if len(op) > 4 else None
            if fused is not None:
                entry.fused = ctypes.addressof(fused)
                self._keep.append(fused)
            self._keep.append(layer)
        handle = c_void_p()
        _lib.call("b200exl3_stack_create", ctypes.cast(table, c_void_p), len(ops), dtype, rows, byref(handle))
        self.handle = handle.value
        self.count, self.rows = len(ops), rows

    def forward(self, stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_stack_forward", c_void_p(self.handle), c_void_p(stream.handle))

    def status(self) -> int:
        out = c_int()
        _lib.call("b200exl3_stack_status", c_void_p(self.handle), byref(out))
        return out.value

    def reset(self) -> None:
        _lib.call("b200exl3_stack_reset", c_void_p(self.handle))

    def geometry(self) -> tuple[int, int]:
        grid, smem = c_int(), c_size_t()
        _lib.call("b200exl3_stack_geometry", c_void_p(self.handle), byref(grid), byref(smem))
        return grid.value, smem.value

    def close(self) -> None:
        if getattr(self, "handle", None):
            _lib.load().b200exl3_stack_free(c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
