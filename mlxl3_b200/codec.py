"""Stand-alone codec and rotation operators over the C ABI, with host arrays in and out.

They mirror the CPU functions of the reference's ``codec`` module (native/src/codec.rs:102-190) and
its rotation chains (native/src/linear.rs:855-861, 978-996), but every value is computed on the GPU.
"""
from __future__ import annotations

from ctypes import c_void_p

import numpy as np

from . import _lib
from ._lib import F16, B200Exl3Error
from .linear import _np_dtype, dtype_code
from .runtime import DEFAULT_STREAM, DeviceBuffer, Stream


def _check_k(k: int) -> None:
    if not 1 <= k <= 8:
        raise B200Exl3Error(f"K must be in 1..=8, got {k}")


def unpack(packed: np.ndarray, k: int, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """packed uint16 (whole tiles of 16*k words) -> 256 uint16 states per tile (``codec::unpack``)."""
    _check_k(k)
    p = np.ascontiguousarray(packed).view(np.uint16).ravel()
    if p.size % (16 * k):
        raise B200Exl3Error("packed length is not a whole tile")
    tiles = p.size // (16 * k)
    if tiles == 0:
        return np.empty(0, np.uint16)
    d_p, d_s = DeviceBuffer.from_numpy(p, stream), DeviceBuffer(tiles * 512)
    _lib.call("b200exl3_unpack_states", c_void_p(d_p.ptr), tiles, k, 0, c_void_p(d_s.ptr), None, c_void_p(stream.handle))
    return d_s.download((tiles * 256,), np.uint16, stream)


def decode_tiles(packed: np.ndarray, k: int, cb: int, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """packed tiles -> fp16 weights in kernel order, 256 per tile."""
    _check_k(k)
    p = np.ascontiguousarray(packed).view(np.uint16).ravel()
    if p.size % (16 * k):
        raise B200Exl3Error("packed length is not a whole tile")
    tiles = p.size // (16 * k)
    if tiles == 0:
        return np.empty(0, np.float16)
    d_p, d_v = DeviceBuffer.from_numpy(p, stream), DeviceBuffer(tiles * 512)
    _lib.call("b200exl3_unpack_states", c_void_p(d_p.ptr), tiles, k, cb, None, c_void_p(d_v.ptr), c_void_p(stream.handle))
    return d_v.download((tiles * 256,), np.float16, stream)


def codebook(states: np.ndarray | None, cb: int, count: int = 65536, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """states -> fp16 weights (``codec::decode_codeword``); ``states=None`` tabulates 0..count-1."""
    if states is None:
        d_s, n = None, count
    else:
        s = np.ascontiguousarray(states, np.uint16).ravel()
        n = s.size
        if n == 0:
            return np.empty(0, np.float16)
        d_s = DeviceBuffer.from_numpy(s, stream)
    d_v = DeviceBuffer(n * 2)
    _lib.call("b200exl3_codebook", c_void_p(d_s.ptr) if d_s else None, n, cb, c_void_p(d_v.ptr), c_void_p(stream.handle))
    return d_v.download((n,), np.float16, stream)


def reconstruct_inner(trellis: np.ndarray, k: int, cb: int, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """trellis [in/16, out/16, 16k] -> fp16 W [in, out] (``codec::reconstruct_inner``)."""
    _check_k(k)
    t = np.ascontiguousarray(trellis).view(np.uint16)
    if t.ndim != 3 or t.shape[2] != 16 * k or min(t.shape) <= 0:
        raise B200Exl3Error("trellis size does not match shape")
    n_in, n_out = t.shape[0] * 16, t.shape[1] * 16
    d_t, d_w = DeviceBuffer.from_numpy(t, stream), DeviceBuffer(n_in * n_out * 2)
    _lib.call("b200exl3_reconstruct", c_void_p(d_t.ptr), n_in, n_out, k, cb, c_void_p(d_w.ptr), c_void_p(stream.handle))
    return d_w.download((n_in, n_out), np.float16, stream)


def prepare(x: np.ndarray, suh: np.ndarray, dtype: int | None = None, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """xhat = H128(half(half(x) * suh)); x [rows, in]; suh [in] or [rows, in] fp16."""
    x = np.ascontiguousarray(x)
    code = dtype_code(x, dtype)
    if x.ndim != 2 or x.shape[1] % 128:
        raise B200Exl3Error("expected complete 128-aligned rows")
    rows, n = x.shape
    s = np.ascontiguousarray(suh, np.float16)
    scale_rows = 1 if s.ndim == 1 else s.shape[0]
    if rows == 0:
        return np.empty((0, n), np.float16)
    d_x, d_s, d_o = DeviceBuffer.from_numpy(x, stream), DeviceBuffer.from_numpy(s, stream), DeviceBuffer(rows * n * 2)
    _lib.call("b200exl3_prepare", c_void_p(d_x.ptr), code, c_void_p(d_s.ptr), scale_rows, rows, n, c_void_p(d_o.ptr),
              c_void_p(stream.handle))
    return d_o.download((rows, n), np.float16, stream)


def finish(partials: np.ndarray, svh: np.ndarray, bias: np.ndarray | None = None, y_dtype: int = F16,
           stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """y = half(H128(half(sum over splits))) * svh (+ bias); partials fp32 [splits, rows, out] or [rows, out]."""
    p = np.ascontiguousarray(partials, np.float32)
    if p.ndim == 2:
        p = p[None]
    splits, rows, n = p.shape
    if n % 128:
        raise B200Exl3Error("expected complete 128-aligned rows")
    s = np.ascontiguousarray(svh, np.float16)
    scale_rows = 1 if s.ndim == 1 else s.shape[0]
    out_dtype = _np_dtype(y_dtype)
    if rows == 0:
        return np.empty((0, n), out_dtype)
    d_p, d_s = DeviceBuffer.from_numpy(p, stream), DeviceBuffer.from_numpy(s, stream)
    d_b = DeviceBuffer.from_numpy(np.ascontiguousarray(bias, np.float16), stream) if bias is not None else None
    d_y = DeviceBuffer(rows * n * np.dtype(out_dtype).itemsize)
    _lib.call("b200exl3_finish", c_void_p(d_p.ptr), splits, c_void_p(d_s.ptr), scale_rows, c_void_p(d_b.ptr) if d_b else None,
              rows, n, y_dtype, c_void_p(d_y.ptr), c_void_p(stream.handle))
    return d_y.download((rows, n), out_dtype, stream)


def permutation() -> np.ndarray:
    """Kernel-order index -> position ``row * 16 + col`` in the 16x16 tile (``codec::permutation``,
    native/src/codec.rs:126-138): lane ``L`` of a warp owns indices ``8L..8L+7`` = rows ``2q + {0, 1, 8, 9}``
    (q = L % 4) of columns ``g`` and ``g + 8`` (g = L // 4), the ``mma.m16n8k16`` fragment order."""
    lane = np.arange(32)[:, None, None]
    rows = (lane % 4) * 2 + np.array([0, 1, 8, 9])[None, None, :]
    cols = lane // 4 + np.array([0, 8])[None, :, None]
    return (rows * 16 + cols).reshape(256)


def permutation_inverse() -> np.ndarray:
    """Tile position -> kernel-order index (``codec::permutation_inverse``, native/src/codec.rs:150-156)."""
    out = np.empty(256, np.int64)
    out[permutation()] = np.arange(256)
    return out


def pack(states: np.ndarray, k: int) -> np.ndarray:
    """States -> packed tiles on the host (``codec::pack``, native/src/codec.rs:72-100): the low ``k`` bits of
    state ``t`` are bits ``[t*k, (t+1)*k)`` of the tile's 256*k-bit stream, most significant bit first; the
    stream is stored as little-endian 32-bit words, i.e. 16-bit group ``l`` of the stream lands at index
    ``l ^ 1``.  Only the quantizer side needs this; it lives here so that the codec tool is complete."""
    _check_k(k)
    s = np.ascontiguousarray(states, np.uint16).reshape(-1)
    if s.size % 256:
        raise B200Exl3Error("encoded length must be a multiple of 256")
    tiles = s.reshape(-1, 256)
    shifts = np.arange(k - 1, -1, -1, dtype=np.uint16)
    bits = ((tiles[:, :, None] >> shifts) & 1).astype(np.uint8).reshape(tiles.shape[0], 256 * k)
    weights = (1 << np.arange(15, -1, -1)).astype(np.uint32)
    groups = (bits.reshape(tiles.shape[0], 16 * k, 16) * weights).sum(axis=2).astype(np.uint16)
    out = np.empty_like(groups)
    out[:, np.arange(16 * k) ^ 1] = groups
    return out.reshape(-1)
