"""``Exl3Linear`` -- the host-side mirror of the reference's quantized-linear operator
(native/src/linear.rs:424-1236 of the reference) over the C ABI.

Same construction arguments, the same validation and error wording, the same ``forward``
contract: ``x`` of any rank with last dimension ``in`` and dtype f16 / f32 (bf16 as uint16 bits with
``dtype=BF16``) gives ``y`` with the same leading dimensions and the same dtype.  All arithmetic
runs in the CUDA library; there is no CPU path.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_size_t, c_void_p

import numpy as np

from . import _lib
from ._lib import BF16, F16, F32, B200Exl3Error
from .runtime import DEFAULT_STREAM, DeviceBuffer, Stream

DEFAULT, MCG, MUL1 = 0, 1, 2


def dtype_code(array: np.ndarray, dtype: int | None = None) -> int:
    if dtype is not None:
        if dtype == BF16 and array.dtype != np.uint16:
            raise B200Exl3Error("bf16 data is passed as uint16 bit patterns")
        return dtype
    if array.dtype == np.float16:
        return F16
    if array.dtype == np.float32:
        return F32
    raise B200Exl3Error(f"unsupported EXL3 input dtype {array.dtype}")


def _np_dtype(code: int):
    return {F16: np.float16, F32: np.float32, BF16: np.uint16}[code]


def _to_f32(array: np.ndarray, code: int) -> np.ndarray:
    if code == BF16:
        return (np.asarray(array, np.uint16).astype(np.uint32) << 16).view(np.float32)
    return np.asarray(array).astype(np.float32)


def _f32_to_bf16_bits(array: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(array, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def new_workspace(nbytes: int) -> DeviceBuffer:
    """Scratch memory for forward calls: its header of arrival counters is zeroed here, once."""
    buf = DeviceBuffer(max(nbytes, _lib.WORKSPACE_HEADER_BYTES))
    _lib.call("b200exl3_memset", c_void_p(buf.ptr), 0, _lib.WORKSPACE_HEADER_BYTES, c_void_p(DEFAULT_STREAM.handle))
    DEFAULT_STREAM.sync()
    return buf


def workspace_status(workspace: DeviceBuffer) -> int:
    """0 if every kernel that used the workspace completed; 1 if a bounded device-side wait gave up."""
    from ctypes import c_int
    out = c_int()
    _lib.call("b200exl3_workspace_status", c_void_p(workspace.ptr), byref(out))
    return out.value


def static_status(clear: bool = False) -> int:
    """Status word of the library's fixed scratch array (used by ``forward_static_device``) on the current
    device: 0, or the code of a bounded device-side wait that gave up.  Sticky until read with ``clear``."""
    from ctypes import c_int
    out = c_int()
    _lib.call("b200exl3_static_status", byref(out), 1 if clear else 0)
    return out.value


class Prologue(ctypes.Structure):
    """``b200exl3_prologue``: the operators fused in front of a layer's input rotation and behind its output rotation
    (fp16; 1 to 8 rows, the SwiGLU prologue alone any number of rows)."""
    _fields_ = [("kind", ctypes.c_int), ("d_aux", c_void_p), ("d_weight", c_void_p), ("d_sum", c_void_p), ("eps", ctypes.c_float),
                ("d_sumsq", c_void_p), ("epilogue", ctypes.c_int), ("d_residual", c_void_p), ("d_residual_out", c_void_p),
                ("d_sumsq_out", c_void_p), ("d_pos", c_void_p), ("theta", ctypes.c_float), ("max_ctx", ctypes.c_int),
                ("d_k_cache", c_void_p), ("d_v_cache", c_void_p)]

    @classmethod
    def rms_norm(cls, d_weight: int, eps: float, d_residual: int = 0, d_sum: int = 0) -> "Prologue":
        """Every warp adds up the whole row (+ residual) itself."""
        return cls(1, d_residual or None, d_weight, d_sum or None, eps)

    @classmethod
    def rms_norm_from_blocks(cls, d_weight: int, eps: float, d_sumsq: int) -> "Prologue":
        """The row's sums of squares per 128-block were left by the residual epilogue of the layer before."""
        return cls(3, None, d_weight, None, eps, d_sumsq)

    @classmethod
    def swiglu(cls, d_up: int) -> "Prologue":
        return cls(2, d_up, None, None, 0.0)

    @classmethod
    def plain(cls) -> "Prologue":
        return cls(0)

    def with_residual(self, d_residual: int, d_residual_out: int, d_sumsq_out: int) -> "Prologue":
        """Adds the residual epilogue: output + residual -> d_residual_out, block sums of squares -> d_sumsq_out."""
        self.epilogue, self.d_residual, self.d_residual_out, self.d_sumsq_out = 1, d_residual, d_residual_out, d_sumsq_out
        return self

    def with_rope(self, d_pos: int, theta: float, max_ctx: int, d_k_cache: int, d_v_cache: int) -> "Prologue":
        """Adds the rotary epilogue of a [q | k | v] group (one row, 128-wide heads): q is rotated into the group's first
        output, k is rotated and v copied into row ``*d_pos`` of the caches."""
        self.epilogue, self.d_pos, self.theta, self.max_ctx = 2, d_pos, theta, max_ctx
        self.d_k_cache, self.d_v_cache = d_k_cache, d_v_cache
        return self


class Exl3Linear:
    """One EXL3-quantized linear layer resident on the GPU.

    ``Exl3Linear(trellis, suh, svh, bias, k, cb)`` follows ``Exl3Linear::new``
    (native/src/linear.rs:577-639): ``trellis`` is ``[in/16, out/16, 16*k]`` int16/uint16, ``suh`` is
    ``[in]``, ``svh`` and the optional ``bias`` are ``[out]`` (f16 or f32; bf16 as uint16 with
    ``scale_dtype=BF16``), ``k`` in 1..8 and ``cb`` one of DEFAULT / MCG / MUL1.
    """

    def __init__(self, trellis: np.ndarray, suh: np.ndarray, svh: np.ndarray, bias: np.ndarray | None, k: int,
                 cb: int = DEFAULT, *, scale_dtype: int | None = None, exact_weights: bool = False):
        if not 1 <= k <= 8:
            raise B200Exl3Error(f"K must be in 1..=8, got {k}")
        if cb not in (DEFAULT, MCG, MUL1):
            raise B200Exl3Error(f"invalid EXL3 codebook {cb}")
        trellis = np.asarray(trellis)
        if trellis.ndim != 3 or trellis.shape[2] != 16 * k or min(trellis.shape) <= 0:
            raise B200Exl3Error("invalid trellis shape")
        rows, cols = trellis.shape[0] * 16, trellis.shape[1] * 16
        if rows % 128 or cols % 128:
            raise B200Exl3Error("public EXL3 projections require 128-aligned dimensions")
        suh, svh = np.asarray(suh), np.asarray(svh)
        if suh.shape != (rows,) or svh.shape != (cols,):
            raise B200Exl3Error("EXL3 scales have wrong dimensions")
        if bias is not None and np.asarray(bias).shape != (cols,):
            raise B200Exl3Error("EXL3 bias has wrong dimensions")
        if trellis.dtype not in (np.uint16, np.int16):
            raise B200Exl3Error("EXL3 trellis must contain 16-bit integers")
        code = dtype_code(suh, scale_dtype)
        cast = _np_dtype(code)
        self.rows, self.cols, self.k, self.cb = rows, cols, k, cb
        d_trellis = DeviceBuffer.from_numpy(trellis.view(np.uint16))
        d_suh = DeviceBuffer.from_numpy(suh.astype(cast, copy=False))
        d_svh = DeviceBuffer.from_numpy(svh.astype(cast, copy=False))
        d_bias = DeviceBuffer.from_numpy(np.asarray(bias).astype(cast, copy=False)) if bias is not None else None
        handle = c_void_p()
        flags = _lib.EXACT_WEIGHTS if exact_weights else 0
        _lib.call("b200exl3_linear_create", c_void_p(d_trellis.ptr), c_void_p(d_suh.ptr), c_void_p(d_svh.ptr),
                  c_void_p(d_bias.ptr) if d_bias else None, code, rows, cols, k, cb, flags, byref(handle))
        self.handle = handle.value
        self._workspace: DeviceBuffer | None = None

    @classmethod
    def from_checkpoint(cls, checkpoint, prefix: str, **options) -> "Exl3Linear":
        """``Exl3Linear::from_checkpoint`` (native/src/linear.rs:454-575): ``{prefix}.trellis``, scales
        ``suh``/``svh`` or their legacy names ``su``/``sv``, the codebook from the presence of ``{prefix}.mul1``
        or ``{prefix}.mcg``, an optional ``{prefix}.bias`` (converted to fp16), K from the trellis' last axis.
        ``checkpoint`` comes from :func:`mlxl3_b200.checkpoint.inspect`."""
        trellis = checkpoint.array(f"{prefix}.trellis")
        if trellis.ndim == 0 or trellis.shape[-1] % 16:
            raise B200Exl3Error("trellis must have dimensions")
        codes = {"F16": F16, "BF16": BF16, "F32": F32}

        def load(name):
            info = checkpoint.tensors.get(name)
            if info is None:
                raise B200Exl3Error(f"missing tensor {name}")
            if info.dtype not in codes:
                raise B200Exl3Error(f"invalid scale dtype {name}")
            return checkpoint.array(name), codes[info.dtype]
        scales = [load(checkpoint.scale_name(prefix, primary, legacy)) for primary, legacy in (("suh", "su"), ("svh", "sv"))]
        bias = None
        if f"{prefix}.bias" in checkpoint.tensors:
            bias = _to_f32(*load(f"{prefix}.bias")).astype(np.float16)          # the reference stores the bias as fp16
        code = scales[0][1]
        if scales[1][1] != code or (bias is not None and code == BF16):
            # the device side takes one dtype for a layer's vectors: widen all of them to fp32 (exact)
            scales = [(_to_f32(a, c), F32) for a, c in scales]
            code = F32
        if bias is not None and code == F32:
            bias = bias.astype(np.float32)
        scales = [a for a, _ in scales]
        return cls(trellis, scales[0], scales[1], bias, trellis.shape[-1] // 16, checkpoint.codebook(prefix),
                   scale_dtype=code, **options)

    # ---- reference accessors (native/src/linear.rs:655-660) ---------------------------------------
    def input_dims(self) -> int:
        return self.rows

    def output_dims(self) -> int:
        return self.cols

    def workspace_bytes(self, rows: int) -> int:
        out = c_size_t()
        _lib.call("b200exl3_linear_workspace_bytes", c_void_p(self.handle), rows, byref(out))
        return out.value

    def _ensure_workspace(self, rows: int) -> DeviceBuffer:
        need = self.workspace_bytes(rows)
        if self._workspace is None or self._workspace.nbytes < need:
            self._workspace = new_workspace(need)
        return self._workspace

    # ---- device-pointer entry points (no host copies) ---------------------------------------------
    def forward_device(self, d_x: int, dtype: int, rows: int, d_y: int, workspace: DeviceBuffer,
                       stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_linear_forward", c_void_p(self.handle), c_void_p(d_x), dtype, rows, c_void_p(d_y),
                  c_void_p(workspace.ptr), workspace.nbytes, c_void_p(stream.handle))

    def forward_fused_device(self, prologue: Prologue, d_x: int, rows: int, d_y: int, workspace: DeviceBuffer,
                             stream: Stream = DEFAULT_STREAM, tp=None) -> None:
        """``forward_device`` for fp16 rows with an RMSNorm or SwiGLU prologue fused into the kernel's input rotation;
        ``tp`` (a ``TpContext``) makes it the row-parallel form."""
        _lib.call("b200exl3_linear_forward_fused", c_void_p(self.handle), byref(prologue), c_void_p(tp.handle) if tp is not None else None,
                  c_void_p(d_x), rows, c_void_p(d_y), c_void_p(workspace.ptr), workspace.nbytes, c_void_p(stream.handle))

    def forward_static_device(self, d_x: int, dtype: int, rows: int, d_y: int, stream: Stream = DEFAULT_STREAM) -> None:
        """``forward_device`` without a workspace: the scratch is a fixed 4 MiB array inside the library,
        for callers that cannot allocate device memory.  Calls must not overlap on the GPU, larger
        scratch needs are refused, and the first call per device must happen outside a graph recording."""
        _lib.call("b200exl3_linear_forward_static", c_void_p(self.handle), c_void_p(d_x), dtype, rows, c_void_p(d_y),
                  c_void_p(stream.handle))

    def forward_partial_device(self, d_x: int, dtype: int, rows: int, d_yhat: int, workspace: DeviceBuffer,
                               stream: Stream = DEFAULT_STREAM) -> None:
        """Input rotation and product only: fp32 ``yhat[rows, out]`` of this (row-parallel) shard."""
        _lib.call("b200exl3_linear_forward_partial", c_void_p(self.handle), c_void_p(d_x), dtype, rows, c_void_p(d_yhat),
                  c_void_p(workspace.ptr), workspace.nbytes, c_void_p(stream.handle))

    def finish_device(self, d_yhat: int, rows: int, dtype: int, d_y: int, stream: Stream = DEFAULT_STREAM) -> None:
        """Output rotation, ``svh`` and bias applied to an (all-reduced) fp32 ``yhat``."""
        _lib.call("b200exl3_linear_finish", c_void_p(self.handle), c_void_p(d_yhat), rows, dtype, c_void_p(d_y),
                  c_void_p(stream.handle))

    # ---- host-buffer entry points (what a caller with numpy arrays uses) --------------------------
    def forward(self, x: np.ndarray, dtype: int | None = None, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        """``Exl3Linear::forward`` (native/src/linear.rs:731-997) with host arrays in and out."""
        x = np.asarray(x)
        if x.ndim == 0 or x.shape[-1] != self.rows:
            raise B200Exl3Error(f"invalid EXL3 linear input for {self.rows} inputs")
        matrix_rows = x.size // self.rows
        if matrix_rows <= 0:
            raise B200Exl3Error("EXL3 linear input cannot be empty")
        code = dtype_code(x, dtype)
        x2 = np.ascontiguousarray(x).reshape(matrix_rows, self.rows)
        d_x = DeviceBuffer.from_numpy(x2, stream)
        d_y = DeviceBuffer(matrix_rows * self.cols * x2.dtype.itemsize)
        self.forward_device(d_x.ptr, code, matrix_rows, d_y.ptr, self._ensure_workspace(matrix_rows), stream)
        y = d_y.download((matrix_rows, self.cols), x2.dtype, stream)
        return y.reshape(*x.shape[:-1], self.cols)

    def forward_raw(self, xhat: np.ndarray, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        """fp32 ``xhat @ W`` for already rotated fp16 inputs ``[rows, in]`` (no rotations, no scales)."""
        xh = np.ascontiguousarray(xhat, np.float16)
        if xh.ndim != 2 or xh.shape[1] != self.rows or xh.shape[0] == 0:
            raise B200Exl3Error(f"invalid EXL3 linear input for {self.rows} inputs")
        rows = xh.shape[0]
        d_x = DeviceBuffer.from_numpy(xh, stream)
        d_y = DeviceBuffer(rows * self.cols * 4)
        ws = self._ensure_workspace(rows)
        _lib.call("b200exl3_linear_forward_raw", c_void_p(self.handle), c_void_p(d_x.ptr), rows, c_void_p(d_y.ptr),
                  c_void_p(ws.ptr), ws.nbytes, c_void_p(stream.handle))
        return d_y.download((rows, self.cols), np.float32, stream)

    def decode(self, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        """Inner matrix ``W[in, out]`` as fp16 (``codec::reconstruct_inner``, native/src/codec.rs:159-190)."""
        d_w = DeviceBuffer(self.rows * self.cols * 2)
        _lib.call("b200exl3_linear_decode", c_void_p(self.handle), c_void_p(d_w.ptr), c_void_p(stream.handle))
        return d_w.download((self.rows, self.cols), np.float16, stream)

    def close(self) -> None:
        if getattr(self, "handle", None):
            _lib.load().b200exl3_linear_free(c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Exl3Group:
    """Projections that read the same input, fused into one launch -- the mirror of the reference's
    ``Exl3Group`` (native/src/linear.rs:2285-2814): ``Exl3Group(linears)`` needs at least two members
    with the same input width, K and codebook; ``forward(x)`` returns one array per member."""

    @staticmethod
    def compatible(linears) -> bool:
        first = linears[0] if linears else None
        return (first is not None and len(linears) >= 2
                and all(l.rows == first.rows and l.k == first.k and l.cb == first.cb for l in linears))

    def __init__(self, linears):
        linears = list(linears)
        if not self.compatible(linears):
            raise B200Exl3Error("incompatible grouped projections")
        self.rows, self.k, self.cb = linears[0].rows, linears[0].k, linears[0].cb
        self.widths = [l.cols for l in linears]
        handles = (c_void_p * len(linears))(*[l.handle for l in linears])
        out = c_void_p()
        _lib.call("b200exl3_group_create", handles, len(linears), byref(out))
        self.handle = out.value
        self._workspace: DeviceBuffer | None = None

    def workspace_bytes(self, rows: int) -> int:
        out = c_size_t()
        _lib.call("b200exl3_group_workspace_bytes", c_void_p(self.handle), rows, byref(out))
        return out.value

    def forward_device(self, d_x: int, dtype: int, rows: int, d_ys, workspace: DeviceBuffer,
                       stream: Stream = DEFAULT_STREAM) -> None:
        ptrs = (c_void_p * len(self.widths))(*d_ys)
        _lib.call("b200exl3_group_forward", c_void_p(self.handle), c_void_p(d_x), dtype, rows, ptrs, c_void_p(workspace.ptr),
                  workspace.nbytes, c_void_p(stream.handle))

    def forward_fused_device(self, prologue: Prologue, d_x: int, rows: int, d_ys, workspace: DeviceBuffer,
                             stream: Stream = DEFAULT_STREAM) -> None:
        ptrs = (c_void_p * len(self.widths))(*d_ys)
        _lib.call("b200exl3_group_forward_fused", c_void_p(self.handle), byref(prologue), c_void_p(d_x), rows, ptrs, c_void_p(workspace.ptr),
                  workspace.nbytes, c_void_p(stream.handle))

    def forward(self, x: np.ndarray, dtype: int | None = None, stream: Stream = DEFAULT_STREAM):
        x = np.asarray(x)
        if x.ndim == 0 or x.shape[-1] != self.rows or x.size == 0:
            raise B200Exl3Error("invalid grouped EXL3 input")
        matrix_rows = x.size // self.rows
        code = dtype_code(x, dtype)
        x2 = np.ascontiguousarray(x).reshape(matrix_rows, self.rows)
        d_x = DeviceBuffer.from_numpy(x2, stream)
        d_ys = [DeviceBuffer(matrix_rows * w * x2.dtype.itemsize) for w in self.widths]
        need = self.workspace_bytes(matrix_rows)
        if self._workspace is None or self._workspace.nbytes < need:
            self._workspace = new_workspace(need)
        self.forward_device(d_x.ptr, code, matrix_rows, [d.ptr for d in d_ys], self._workspace, stream)
        return [d.download((matrix_rows, w), x2.dtype, stream).reshape(*x.shape[:-1], w) for d, w in zip(d_ys, self.widths)]

    def close(self) -> None:
        if getattr(self, "handle", None):
            _lib.load().b200exl3_group_free(c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
