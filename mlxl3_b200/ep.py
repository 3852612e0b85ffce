"""Expert parallelism of the grouped-expert SwiGLU block (one process per GPU).

Rank r of W owns experts ``[r * E / W, (r + 1) * E / W)``: the gate, up and down columns of those experts and their
scale rows.  Token rows, routes and scores are the same on every rank (the router is replicated).  A (token, choice)
slot is computed where its expert lives (dispatch), and every rank adds its rows' slot results in slot order (combine),
exactly as ``finish_and_reduce`` of the reference does on one device (native/src/moe.rs:586-609).
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_size_t, c_void_p

import numpy as np

from . import _lib
from ._lib import B200Exl3Error, F16, F32
from .linear import dtype_code, new_workspace
from .moe import Exl3SwitchGlu
from .runtime import DEFAULT_STREAM, DeviceBuffer, Stream


def expert_range(rank: int, world: int, experts: int) -> tuple[int, int]:
    """(first expert, number of experts) of ``rank``."""
    if world < 1 or experts % world:
        raise ValueError(f"{experts} experts do not split over {world} ranks")
    per = experts // world
    return rank * per, per


def owner_of(selected: np.ndarray, world: int, experts: int) -> np.ndarray:
    """Rank that computes each slot (ids beyond the bank belong to nobody and contribute nothing)."""
    return np.asarray(selected, np.int64) // (experts // world)


def local_plan(selected: np.ndarray, rank: int, world: int, experts: int):
    """(slot indices in ascending order, local expert ids) of the slots ``rank`` computes: the dispatch half."""
    first, per = expert_range(rank, world, experts)
    flat = np.asarray(selected, np.int64).reshape(-1)
    slots = np.nonzero((flat >= first) & (flat < first + per))[0]
    return slots, flat[slots] - first


def shard_bank(gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, rank: int, world: int):
    """The six arrays of ``rank``'s experts.  The gate|up bank keeps the reference's layout (gate columns of all the
    experts, then up columns of all the experts: native/src/moe.rs:754-807), restricted to the local experts."""
    experts, _, n_in = np.asarray(gu_suh).shape
    hidden = np.asarray(gu_svh).shape[2]
    first, per = expert_range(rank, world, experts)
    ht, it = hidden // 16, n_in // 16
    gate = gu_trellis[:, first * ht:(first + per) * ht]
    up = gu_trellis[:, (experts + first) * ht:(experts + first + per) * ht]
    e = slice(first, first + per)
    return (np.ascontiguousarray(np.concatenate([gate, up], axis=1)), np.ascontiguousarray(gu_suh[e]), np.ascontiguousarray(gu_svh[e]),
            np.ascontiguousarray(down_trellis[:, first * it:(first + per) * it]), np.ascontiguousarray(down_suh[e]),
            np.ascontiguousarray(down_svh[e]))


class EpContext:
    """Peer-memory inboxes of one rank (``b200exl3_ep_*``).  ``exchange`` takes this rank's 64-byte handle and returns
    every rank's handle in rank order (for example through ``torch.distributed.all_gather_object``)."""

    def __init__(self, rank: int, world: int, max_slots: int, width: int, exchange):
        self.rank, self.world, self.max_slots, self.width = rank, world, max_slots, width
        nbytes = c_size_t()
        _lib.call("b200exl3_ep_buffer_bytes", max_slots, width, byref(nbytes))
        own = c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.call("b200exl3_ipc_alloc", nbytes.value, byref(own), handle)
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
        _lib.call("b200exl3_ep_create", rank, world, max_slots, width, pointers, byref(ctx))
        self.handle = ctx.value

    def status(self) -> int:
        out = c_int()
        _lib.call("b200exl3_ep_status", c_void_p(self.handle), byref(out))
        return out.value

    def close(self) -> None:
        """Call on every rank after all ranks have finished using the inboxes."""
        if getattr(self, "handle", None):
            _lib.load().b200exl3_ep_free(c_void_p(self.handle))
            self.handle = None
            for peer in self._peers:
                _lib.load().b200exl3_tp_close(c_void_p(peer))
            self._peers = []
            _lib.load().b200exl3_free(c_void_p(self._own))
            self._own = None


class Exl3SwitchGluEp:
    """This rank's share of an ``Exl3SwitchGlu``: ``Exl3SwitchGluEp(bank..., top_k, k, cb, context)`` takes the FULL
    banks (as ``Exl3SwitchGlu`` does) and keeps the rank's experts; ``forward(x, selected, scores)`` has the operator's
    contract and returns the same rows on every rank."""

    def __init__(self, gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, top_k: int, k: int, cb: int, context: EpContext,
                 **options):
        self.context = context
        self.experts = np.asarray(gu_suh).shape[0]
        self.first, per = expert_range(context.rank, context.world, self.experts)
        if per < top_k:
            raise B200Exl3Error("every rank needs at least top_k experts")
        local = shard_bank(gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, context.rank, context.world)
        self.local = Exl3SwitchGlu(*local, top_k, k, cb, **options)
        self.top_k, self.input = top_k, self.local.input
        self._workspace: DeviceBuffer | None = None

    def workspace_bytes(self, rows: int) -> int:
        out = c_size_t()
        _lib.call("b200exl3_moe_ep_workspace_bytes", c_void_p(self.local.handle), rows, byref(out))
        return out.value

    def forward_device(self, d_x: int, x_dtype: int, rows: int, d_selected: int, d_scores: int, score_dtype: int, d_y: int,
                       workspace: DeviceBuffer, stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_moe_forward_ep", c_void_p(self.local.handle), c_void_p(self.context.handle), self.first, c_void_p(d_x), x_dtype,
                  rows, c_void_p(d_selected), c_void_p(d_scores), score_dtype, c_void_p(d_y), c_void_p(workspace.ptr), workspace.nbytes,
                  c_void_p(stream.handle))

    def forward(self, x: np.ndarray, selected: np.ndarray, scores: np.ndarray, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        x, selected, scores = np.asarray(x), np.asarray(selected), np.asarray(scores)
        rows = x.shape[0]
        if x.ndim != 2 or rows <= 0 or x.shape[1] != self.input or selected.shape != (rows, self.top_k) or scores.shape != (rows, self.top_k):
            raise B200Exl3Error("invalid SwitchGLU input/routes")
        if scores.dtype not in (np.float16, np.float32):
            raise B200Exl3Error("routing weights must be float16 or float32")
        d_x = DeviceBuffer.from_numpy(x, stream)
        d_sel = DeviceBuffer.from_numpy(selected.astype(np.uint32, copy=False), stream)
        d_scores = DeviceBuffer.from_numpy(scores, stream)
        d_y = DeviceBuffer(rows * self.input * scores.dtype.itemsize)
        need = self.workspace_bytes(rows)
        if self._workspace is None or self._workspace.nbytes < need:
            self._workspace = new_workspace(need)
        self.forward_device(d_x.ptr, dtype_code(x), rows, d_sel.ptr, d_scores.ptr, F16 if scores.dtype == np.float16 else F32, d_y.ptr,
                            self._workspace, stream)
        return d_y.download((rows, self.input), scores.dtype, stream)

    def close(self) -> None:
        self.local.close()
