"""Host-side mirror of the reference's grouped-expert SwiGLU block ``Exl3SwitchGlu``
(native/src/moe.rs:808-971) over the C ABI (``b200exl3_moe_*``)."""
from __future__ import annotations

from ctypes import byref, c_size_t, c_void_p

import numpy as np

from . import _lib
from ._lib import B200Exl3Error, F16, F32
from .linear import DEFAULT, MCG, MUL1, dtype_code, _np_dtype, new_workspace
from .runtime import DEFAULT_STREAM, DeviceBuffer, Stream


class Exl3SwitchGlu:
    """``Exl3SwitchGlu(gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, top_k, k, cb)`` with the
    shapes ``Exl3SwitchGlu::new`` checks (native/src/moe.rs:808-905): ``gu_suh [experts, 2, in]``,
    ``gu_svh [experts, 2, hidden]``, ``down_suh [experts, hidden]``, ``down_svh [experts, in]``,
    ``gu_trellis [in/16, experts*hidden/8, 16k]`` (gate columns of all experts, then up columns),
    ``down_trellis [hidden/16, experts*in/16, 16k]``.  ``forward(x, selected, scores)`` takes ``x [rows, in]``,
    ``selected [rows, top_k]`` uint32 and ``scores [rows, top_k]`` (f16 or f32) and returns ``[rows, in]`` in the
    dtype of ``scores``."""

    def __init__(self, gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, top_k: int, k: int,
                 cb: int = DEFAULT, *, scale_dtype: int | None = None, exact_weights: bool = False):
        gu_suh, gu_svh = np.asarray(gu_suh), np.asarray(gu_svh)
        down_suh, down_svh = np.asarray(down_suh), np.asarray(down_svh)
        gu_trellis, down_trellis = np.asarray(gu_trellis), np.asarray(down_trellis)
        if gu_suh.ndim != 3:
            raise B200Exl3Error("gate/up input scales must have rank 3")
        if gu_svh.ndim != 3:
            raise B200Exl3Error("gate/up output scales must have rank 3")
        experts, projections, n_in = gu_suh.shape
        hidden = gu_svh.shape[2]
        if (not 1 <= k <= 8 or k == 7 or cb not in (DEFAULT, MCG, MUL1) or experts <= 0 or top_k <= 0 or top_k > experts
                or n_in <= 0 or hidden <= 0 or n_in % 128 or hidden % 128):
            raise B200Exl3Error("invalid or overflowing SwitchGLU dimensions")
        if projections != 2 or gu_svh.shape[:2] != (experts, 2):
            raise B200Exl3Error("invalid SwitchGLU dimensions")
        if (down_suh.shape != (experts, hidden) or down_svh.shape != (experts, n_in)
                or gu_trellis.shape != (n_in // 16, experts * hidden // 8, 16 * k)
                or down_trellis.shape != (hidden // 16, experts * n_in // 16, 16 * k)):
            raise B200Exl3Error("SwitchGLU trellis/scales disagree")
        if any(t.dtype not in (np.uint16, np.int16) for t in (gu_trellis, down_trellis)):
            raise B200Exl3Error("expert trellis must contain 16-bit integers")
        code = dtype_code(gu_suh, scale_dtype)
        cast = _np_dtype(code)
        self.experts, self.input, self.hidden, self.top_k, self.k, self.cb = experts, n_in, hidden, top_k, k, cb
        bufs = [DeviceBuffer.from_numpy(a) for a in (
            gu_trellis.view(np.uint16), gu_suh.astype(cast, copy=False), gu_svh.astype(cast, copy=False),
            down_trellis.view(np.uint16), down_suh.astype(cast, copy=False), down_svh.astype(cast, copy=False))]
        handle = c_void_p()
        _lib.call("b200exl3_moe_create", *(c_void_p(b.ptr) for b in bufs), code, experts, n_in, hidden, top_k, k, cb,
                  _lib.EXACT_WEIGHTS if exact_weights else 0, byref(handle))
        self.handle = handle.value
        self._workspace: DeviceBuffer | None = None

    @classmethod
    def from_checkpoint(cls, checkpoint, prefix: str, experts: int, top_k: int,
                        names=("gate_proj", "up_proj", "down_proj"), **options) -> "Exl3SwitchGlu":
        """``Exl3SwitchGlu::from_checkpoint`` (native/src/moe.rs:629-807): experts ``{prefix}.{e}.{projection}``
        for e in 0..experts; the gate trellises of all experts followed by the up trellises of all experts are
        joined on the output axis, the down trellises likewise; scales are stacked per expert.  All experts must
        share one bit width and one codebook.  ``names=("w1", "w3", "w2")`` reads the LFM naming."""
        if not (experts > 0 and 0 < top_k <= experts and experts <= len(checkpoint.tensors) // 3):
            raise B200Exl3Error("invalid expert count or incomplete expert bank")
        gate, up, down = ([f"{prefix}.{e}.{projection}" for e in range(experts)] for projection in names)
        k = cb = None
        for name in gate + up + down:
            info = checkpoint.tensors.get(f"{name}.trellis")
            if info is None:
                raise B200Exl3Error(f"missing expert trellis {name}")
            if info.dtype not in ("I16", "U16"):
                raise B200Exl3Error(f"{name}: expert trellis must contain 16-bit integers")
            if not info.shape:
                raise B200Exl3Error("empty expert trellis")
            bits = info.shape[-1] // 16
            if k is not None and k != bits:
                raise B200Exl3Error("mixed expert bit widths")
            mode = checkpoint.codebook(name)
            if cb is not None and cb != mode:
                raise B200Exl3Error("mixed expert codebooks")
            k, cb = bits, mode

        def trellises(group):
            # signed and unsigned trellis words carry bits, never numeric values
            return [checkpoint.array(f"{name}.trellis").view(np.uint16) for name in group]

        def scales(group, primary, legacy):
            out = []
            for name in group:
                key = checkpoint.scale_name(name, primary, legacy)
                info = checkpoint.tensors.get(key)
                if info is None:
                    raise B200Exl3Error(f"missing tensor {key}")
                code = {"F16": F16, "BF16": 12, "F32": F32}.get(info.dtype)
                if code is None:
                    raise B200Exl3Error(f"invalid scale dtype {key}")
                a = checkpoint.array(key)
                out.append((a.astype(np.uint32) << 16).view(np.float32) if code == 12 else a.astype(np.float32))
            return np.stack(out)

        gu_trellis = np.concatenate(trellises(gate) + trellises(up), axis=1)
        down_trellis = np.concatenate(trellises(down), axis=1)
        gu_suh = np.stack([scales(gate, "suh", "su"), scales(up, "suh", "su")], axis=1)
        gu_svh = np.stack([scales(gate, "svh", "sv"), scales(up, "svh", "sv")], axis=1)
        return cls(gu_trellis, gu_suh, gu_svh, down_trellis, scales(down, "suh", "su"), scales(down, "svh", "sv"),
                   top_k, k, cb, **options)

    def workspace_bytes(self, rows: int) -> int:
        out = c_size_t()
        _lib.call("b200exl3_moe_workspace_bytes", c_void_p(self.handle), rows, byref(out))
        return out.value

    def forward_device(self, d_x: int, x_dtype: int, rows: int, d_selected: int, d_scores: int, score_dtype: int, d_y: int,
                       workspace: DeviceBuffer, stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_moe_forward", c_void_p(self.handle), c_void_p(d_x), x_dtype, rows, c_void_p(d_selected),
                  c_void_p(d_scores), score_dtype, c_void_p(d_y), c_void_p(workspace.ptr), workspace.nbytes,
                  c_void_p(stream.handle))

    def forward(self, x: np.ndarray, selected: np.ndarray, scores: np.ndarray, dtype: int | None = None,
                stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        """``Exl3SwitchGlu::forward`` (native/src/moe.rs:905-971) with host arrays in and out."""
        x, selected, scores = np.asarray(x), np.asarray(selected), np.asarray(scores)
        if x.ndim != 2:
            raise B200Exl3Error("SwitchGLU input must have rank 2")
        rows = x.shape[0]
        if (rows <= 0 or x.shape[1] != self.input or selected.shape != (rows, self.top_k)
                or scores.shape != (rows, self.top_k)):
            raise B200Exl3Error("invalid SwitchGLU input/routes")
        if scores.dtype not in (np.float16, np.float32):
            raise B200Exl3Error("routing weights must be float16 or float32")
        score_code = F16 if scores.dtype == np.float16 else F32
        d_x = DeviceBuffer.from_numpy(x, stream)
        d_sel = DeviceBuffer.from_numpy(selected.astype(np.uint32, copy=False), stream)
        d_scores = DeviceBuffer.from_numpy(scores, stream)
        d_y = DeviceBuffer(rows * self.input * scores.dtype.itemsize)
        need = self.workspace_bytes(rows)
        if self._workspace is None or self._workspace.nbytes < need:
            self._workspace = new_workspace(need)
        self.forward_device(d_x.ptr, dtype_code(x, dtype), rows, d_sel.ptr, d_scores.ptr, score_code, d_y.ptr,
                            self._workspace, stream)
        return d_y.download((rows, self.input), scores.dtype, stream)

    def close(self) -> None:
        if getattr(self, "handle", None):
            _lib.load().b200exl3_moe_free(c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def expert_mapped(x: np.ndarray, trellis: np.ndarray, suh, svh, selected: np.ndarray, output_dims: int, projections_per_route: int,
                  projection_stride_tiles: int, k: int, cb: int = DEFAULT, input_pretransformed: bool = False, return_raw: bool = False,
                  stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """``expert_mapped`` (native/src/linear.rs:2817-2851): ``x [slots * projections, in]`` (fp16), a bank trellis
    ``[in/16, source_tiles, 16k]``, per-row scales ``suh [rows, in]`` / ``svh [rows, out]`` (``None`` where unused),
    ``selected [slots]`` uint32 -> fp32 raw products or fp16 rotated outputs ``[rows, output_dims]``."""
    x = np.ascontiguousarray(x, np.float16)
    trellis = np.ascontiguousarray(trellis).view(np.uint16)
    selected = np.ascontiguousarray(selected, np.uint32).reshape(-1)
    rows, n_in = x.shape
    if selected.size == 0 or rows != selected.size * projections_per_route:
        raise B200Exl3Error("missing expert routes")
    if trellis.ndim != 3 or trellis.shape[0] * 16 != n_in or trellis.shape[2] != 16 * k:
        raise B200Exl3Error("invalid expert trellis dimensions")
    bufs = [DeviceBuffer.from_numpy(a, stream) for a in (x, trellis, selected)]
    d_suh = DeviceBuffer.from_numpy(np.ascontiguousarray(suh, np.float16), stream) if suh is not None else None
    d_svh = DeviceBuffer.from_numpy(np.ascontiguousarray(svh, np.float16), stream) if svh is not None else None
    d_out = DeviceBuffer(rows * output_dims * (4 if return_raw else 2))
    _lib.call("b200exl3_expert_mapped", c_void_p(bufs[0].ptr), F16, c_void_p(bufs[1].ptr), trellis.shape[1],
              c_void_p(d_suh.ptr) if d_suh else None, c_void_p(d_svh.ptr) if d_svh else None, c_void_p(bufs[2].ptr), selected.size, n_in,
              output_dims, projections_per_route, projection_stride_tiles, k, cb, int(input_pretransformed), int(return_raw),
              c_void_p(d_out.ptr), c_void_p(stream.handle))
    return d_out.download((rows, output_dims), np.float32 if return_raw else np.float16, stream)


def swiglu_down_input(state: np.ndarray, gu_svh: np.ndarray, down_suh: np.ndarray, selected: np.ndarray,
                      stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """``moe::swiglu_down_input`` (native/src/moe.rs:438-533): raw gate/up products ``[slots * 2, hidden]`` fp32 ->
    rotated down-projection inputs ``[slots, hidden]`` fp16."""
    state = np.ascontiguousarray(state, np.float32)
    gu_svh, down_suh = np.ascontiguousarray(gu_svh, np.float16), np.ascontiguousarray(down_suh, np.float16)
    selected = np.ascontiguousarray(selected, np.uint32).reshape(-1)
    hidden = state.shape[1]
    if state.shape[0] != 2 * selected.size or gu_svh.shape[1:] != (2, hidden) or down_suh.shape != (gu_svh.shape[0], hidden):
        raise B200Exl3Error("invalid gate/up scales")
    bufs = [DeviceBuffer.from_numpy(a, stream) for a in (state, gu_svh, down_suh, selected)]
    d_out = DeviceBuffer(selected.size * hidden * 2)
    _lib.call("b200exl3_swiglu_down_input", *(c_void_p(b.ptr) for b in bufs), gu_svh.shape[0], selected.size, hidden, c_void_p(d_out.ptr),
              c_void_p(stream.handle))
    return d_out.download((selected.size, hidden), np.float16, stream)


def finish_and_reduce(state: np.ndarray, svh_rows: np.ndarray, scores: np.ndarray, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """``moe::finish_and_reduce`` (native/src/moe.rs:586-609): raw down products ``[rows * top_k, width]`` fp32, the
    output scales of every slot ``[rows * top_k, width]`` and ``scores [rows, top_k]`` -> ``[rows, width]``."""
    state = np.ascontiguousarray(state, np.float32)
    svh_rows = np.ascontiguousarray(svh_rows, np.float16)
    scores = np.ascontiguousarray(scores)
    if scores.dtype not in (np.float16, np.float32) or scores.ndim != 2 or state.shape != svh_rows.shape or state.shape[0] != scores.size:
        raise B200Exl3Error("invalid expert reduction input")
    rows, top_k = scores.shape
    slots, width = state.shape
    every = np.arange(slots, dtype=np.uint32)                      # each slot has its own row of scales
    bufs = [DeviceBuffer.from_numpy(a, stream) for a in (state, svh_rows, every, scores)]
    d_y = DeviceBuffer(rows * width * scores.dtype.itemsize)
    _lib.call("b200exl3_finish_and_reduce", c_void_p(bufs[0].ptr), c_void_p(bufs[1].ptr), c_void_p(bufs[2].ptr), slots, c_void_p(bufs[3].ptr),
              F16 if scores.dtype == np.float16 else F32, rows, top_k, width, c_void_p(d_y.ptr), c_void_p(stream.handle))
    return d_y.download((rows, width), scores.dtype, stream)
