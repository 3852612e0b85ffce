"""Vectorised numpy restatement of the EXL3 format and rotation arithmetic.

TEST INFRASTRUCTURE ONLY -- a second, independent statement of the same rules as
``exl3_oracle.c`` so the two can be checked against each other and against the
reference's golden vectors.  Parity status: pinned by those vectors.

Reference locations (paths inside the reference project):
  native/src/codec.rs:40-71, 102-138, 159-190   window, codebooks, unpack, permutation, reconstruct
  native/shaders/exl3.metal:156-170             Hadamard-128 rounding points
  native/src/linear.rs:855-861, 978-996         input / output rotation chains
"""
from __future__ import annotations

import numpy as np

HAD_SCALE = np.array([0x3DB504F3], np.uint32).view(np.float32)[0]


def decode_codewords(states: np.ndarray, cb: int) -> np.ndarray:
    """uint16 states -> fp16 weights (native/src/codec.rs:52-71)."""
    x = np.asarray(states).astype(np.uint64)
    if cb == 2:
        b = (x * 0x83DCD12D) & 0xFFFFFFFF
        s = 0x6400 + (b & 255) + ((b >> 8) & 255) + ((b >> 16) & 255) + (b >> 24)
        h = s.astype(np.uint16).view(np.float16).astype(np.float64)
        inv = np.array([0x1EEE], np.uint16).view(np.float16).astype(np.float64)[0]
        bias = np.array([0xC931], np.uint16).view(np.float16).astype(np.float64)[0]
        return (h * inv + bias).astype(np.float16)          # exact in f64, one rounding
    b = (x * 89226354 + 64248484) & 0xFFFFFFFF if cb == 0 else (x * 0xCBAC1FED) & 0xFFFFFFFF
    b = 0x3B603B60 ^ (b & 0x8FFF8FFF)
    lo = (b & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    hi = (b >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    return (lo + hi).astype(np.float16)                     # fp32 sum is exact here


def unpack(packed: np.ndarray, k: int) -> np.ndarray:
    """[..., 16k] uint16 -> [..., 256] uint16 states (native/src/codec.rs:40-46, 102-124)."""
    p = np.ascontiguousarray(packed, dtype=np.uint16)
    words = (p[..., 0::2].astype(np.uint64) | (p[..., 1::2].astype(np.uint64) << 16))
    t = np.arange(256)
    b0 = t * k + k + 256 * k - 16
    b1 = b0 + 16
    i0 = (b0 // 32) % (8 * k)
    last = (b1 - 1) // 32
    i1 = last % (8 * k)
    shift = ((last + 1) * 32 - b1).astype(np.uint64)
    merged = (words[..., i0] << np.uint64(32)) | words[..., i1]
    return ((merged >> shift) & np.uint64(0xFFFF)).astype(np.uint16)


def pack(states: np.ndarray, k: int) -> np.ndarray:
    """[..., 256] states (low k bits used) -> [..., 16k] uint16 (native/src/codec.rs:34-38, 73-100)."""
    s = np.asarray(states).astype(np.uint32)
    fresh = s & ((1 << k) - 1)
    bits = ((fresh[..., :, None] >> np.arange(k - 1, -1, -1)) & 1).reshape(*s.shape[:-1], 256 * k)
    w16 = bits.reshape(*s.shape[:-1], 16 * k, 16)
    vals = (w16 << np.arange(15, -1, -1)).sum(-1).astype(np.uint16)
    out = np.empty_like(vals)
    out[..., 0::2] = vals[..., 1::2]
    out[..., 1::2] = vals[..., 0::2]
    return out


def permutation() -> np.ndarray:
    """kernel-order index -> row*16+col (native/src/codec.rs:126-138)."""
    out = np.zeros(256, np.int64)
    for lane in range(32):
        r, c = (lane % 4) * 2, lane // 4
        for cg in range(2):
            for ri, row in enumerate((r, r + 1, r + 8, r + 9)):
                out[lane * 8 + cg * 4 + ri] = row * 16 + c + 8 * cg
    return out


def reconstruct_inner(trellis: np.ndarray, k: int, cb: int) -> np.ndarray:
    """[in/16, out/16, 16k] -> fp16 W[in, out] (native/src/codec.rs:159-190)."""
    tk, tn, _ = trellis.shape
    vals = decode_codewords(unpack(trellis, k), cb)          # [tk, tn, 256] kernel order
    tiles = np.empty((tk, tn, 256), np.float16)
    tiles[..., permutation()] = vals
    return tiles.reshape(tk, tn, 16, 16).transpose(0, 2, 1, 3).reshape(tk * 16, tn * 16)


def _had_stage(v: np.ndarray, stride: int) -> np.ndarray:
    shp = v.shape
    w = v.reshape(*shp[:-1], 128 // (2 * stride), 2, stride)
    a, b = w[..., 0, :], w[..., 1, :]
    return np.stack([a + b, a - b], axis=-2).reshape(shp)


def hadamard128(x: np.ndarray, round_mid: bool = True, round_end: bool = True, scale: bool = True) -> np.ndarray:
    """fp16 [..., 128] -> fp16; fp32 butterflies, fp16 rounding after strides 8 and 64, then * 2^-3.5."""
    v = np.asarray(x, np.float16).astype(np.float32)
    for stride in (1, 2, 4, 8, 16, 32, 64):
        v = _had_stage(v, stride)
        if (stride == 8 and round_mid) or (stride == 64 and round_end):
            v = v.astype(np.float16).astype(np.float32)
    if scale:
        v = v * HAD_SCALE
    return v.astype(np.float16)


def prepare(x: np.ndarray, suh: np.ndarray) -> np.ndarray:
    """xhat = H128(half(half(x) * suh)) per 128-block (native/src/linear.rs:855-861)."""
    p = np.asarray(x).astype(np.float16) * np.asarray(suh, np.float16)
    return hadamard128(p.reshape(*p.shape[:-1], -1, 128)).reshape(p.shape)


def finish(yhat: np.ndarray, svh: np.ndarray) -> np.ndarray:
    """y = half(H128(half(yhat)) * svh) (native/src/linear.rs:984-989), fp16 result."""
    p = np.asarray(yhat, np.float32).astype(np.float16)
    r = hadamard128(p.reshape(*p.shape[:-1], -1, 128)).reshape(p.shape)
    return r * np.asarray(svh, np.float16)


def linear_forward(trellis, k, cb, suh, svh, x, acc=np.float32) -> np.ndarray:
    """Whole chain with a dense matmul over the decoded matrix (accumulation order: numpy's)."""
    w = reconstruct_inner(trellis, k, cb).astype(acc)
    xh = prepare(x, suh).astype(acc)
    return finish((xh @ w).astype(np.float32), svh)
