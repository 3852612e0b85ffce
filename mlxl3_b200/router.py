"""Stable MoE top-k (``router::topk``, native/src/router.rs:37-120) over the C ABI."""
from __future__ import annotations

from ctypes import c_void_p

import numpy as np

from . import _lib
from ._lib import B200Exl3Error, F16, F32
from .runtime import DEFAULT_STREAM, DeviceBuffer, Stream


def topk_device(d_values: int, dtype: int, rows: int, experts: int, top_k: int, normalize: bool, d_indices: int,
                d_scores: int, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_router_topk", c_void_p(d_values), dtype, rows, experts, top_k, int(normalize), c_void_p(d_indices),
              c_void_p(d_scores), c_void_p(stream.handle))


def topk(values: np.ndarray, top_k: int, normalize: bool, stream: Stream = DEFAULT_STREAM):
    """``values [rows, experts]`` (float16 or float32) -> ``(indices [rows, top_k] uint32, scores [rows, top_k])``:
    per row the ``top_k`` largest values in ascending order, ties to the higher index; with ``normalize`` the
    scores are divided by their sum (added in slot order in the values' dtype)."""
    values = np.asarray(values)
    if values.ndim != 2:
        raise B200Exl3Error("router values must have rank 2")
    if values.dtype not in (np.float16, np.float32):
        raise B200Exl3Error("native router expects FP16 or FP32 values")
    rows, experts = values.shape
    d_values = DeviceBuffer.from_numpy(values, stream)
    d_indices = DeviceBuffer(max(rows * top_k, 1) * 4)
    d_scores = DeviceBuffer(max(rows * top_k, 1) * values.dtype.itemsize)
    topk_device(d_values.ptr, F16 if values.dtype == np.float16 else F32, rows, experts, top_k, normalize, d_indices.ptr,
                d_scores.ptr, stream)
    return (d_indices.download((rows, top_k), np.uint32, stream), d_scores.download((rows, top_k), values.dtype, stream))


def softmax_topk(logits: np.ndarray, top_k: int, normalize: bool = True, stream: Stream = DEFAULT_STREAM):
    """``router::topk(&logits.softmax_precise(), top_k, normalize)`` (native/src/qwen35.rs:214): returns
    ``(indices, scores, probabilities)``; the softmax runs in fp32 and is rounded to the logits' dtype."""
    logits = np.asarray(logits)
    if logits.ndim != 2:
        raise B200Exl3Error("router values must have rank 2")
    if logits.dtype not in (np.float16, np.float32):
        raise B200Exl3Error("native router expects FP16 or FP32 values")
    rows, experts = logits.shape
    d_logits = DeviceBuffer.from_numpy(logits, stream)
    d_indices = DeviceBuffer(max(rows * top_k, 1) * 4)
    d_scores = DeviceBuffer(max(rows * top_k, 1) * logits.dtype.itemsize)
    d_probs = DeviceBuffer(max(logits.nbytes, 1))
    _lib.call("b200exl3_router_softmax_topk", c_void_p(d_logits.ptr), F16 if logits.dtype == np.float16 else F32, rows, experts,
              top_k, int(normalize), c_void_p(d_indices.ptr), c_void_p(d_scores.ptr), c_void_p(d_probs.ptr), c_void_p(stream.handle))
    return (d_indices.download((rows, top_k), np.uint32, stream), d_scores.download((rows, top_k), logits.dtype, stream),
            d_probs.download((rows, experts), logits.dtype, stream))


def gate(x: np.ndarray, weight: np.ndarray, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
    """fp16 router logits ``x [rows, in] @ weight [experts, in].T`` with fp32 accumulation."""
    x, weight = np.ascontiguousarray(x, np.float16), np.ascontiguousarray(weight, np.float16)
    if x.ndim != 2 or weight.ndim != 2 or x.shape[1] != weight.shape[1]:
        raise B200Exl3Error("invalid router gate dimensions")
    rows, n_in = x.shape
    experts = weight.shape[0]
    d_x, d_w = DeviceBuffer.from_numpy(x, stream), DeviceBuffer.from_numpy(weight, stream)
    d_logits = DeviceBuffer(rows * experts * 2)
    _lib.call("b200exl3_router_gate", c_void_p(d_x.ptr), F16, c_void_p(d_w.ptr), rows, n_in, experts, c_void_p(d_logits.ptr),
              c_void_p(stream.handle))
    return d_logits.download((rows, experts), np.float16, stream)
