"""CPU oracle for the EXL3 quantized-linear path.  TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference's arithmetic live here:

* ``exl3_oracle.c``  -- plain C, threaded; loaded through :func:`lib` (ctypes).
* ``exl3_numpy.py``  -- vectorised numpy.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package.  The shipped library never does: it has no CPU path.

Parity status: pinned (see the header of ``exl3_oracle.c``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

F16, F32, BF16 = 9, 10, 12

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libexl3oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``exl3_oracle.c`` with the Makefile beside it."""
    src = _HERE / "exl3_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    try:
        L = ctypes.CDLL(str(_SO))
    except OSError:
        build(force=True)
        L = ctypes.CDLL(str(_SO))
    c_i, c_i64, c_sz, c_p = ctypes.c_int, ctypes.c_int64, ctypes.c_size_t, ctypes.c_void_p
    L.exl3o_decode_codeword.restype = ctypes.c_uint16
    L.exl3o_decode_codeword.argtypes = [ctypes.c_uint16, c_i]
    L.exl3o_codebook_table.restype = None
    L.exl3o_codebook_table.argtypes = [c_i, c_p]
    L.exl3o_pack.argtypes = [c_p, c_sz, c_i, c_p]
    L.exl3o_unpack.argtypes = [c_p, c_sz, c_i, c_p]
    L.exl3o_permutation.restype = None
    L.exl3o_permutation.argtypes = [c_p]
    L.exl3o_permutation_inverse.restype = None
    L.exl3o_permutation_inverse.argtypes = [c_p]
    L.exl3o_reconstruct_inner.argtypes = [c_p, c_i, c_i, c_i, c_i, c_p, c_i]
    L.exl3o_hadamard128.restype = None
    L.exl3o_hadamard128.argtypes = [c_p, c_p, c_sz]
    L.exl3o_prepare.argtypes = [c_p, c_i, c_p, c_i64, c_i64, c_i, c_p]
    L.exl3o_finish.argtypes = [c_p, c_p, c_i64, c_p, c_i64, c_i, c_i, c_p]
    L.exl3o_matmul_raw.argtypes = [c_p, c_i, c_i, c_i, c_i, c_p, c_i64, c_i, c_i, c_i, c_p, c_i]
    L.exl3o_linear_forward.argtypes = [c_p, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_i64, c_p, c_i]
    L.exl3o_glu_down_input.argtypes = [c_p, c_p, c_p, c_p, c_p, c_i64, c_i, c_p]
    L.exl3o_finish_and_reduce.argtypes = [c_p, c_p, c_p, c_i64, c_i, c_i, c_p]
    _lib = L
    return L


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _u16(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype == np.float16 or a.dtype == np.int16:
        a = a.view(np.uint16)
    return np.ascontiguousarray(a, dtype=np.uint16)


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    if dt == np.float16:
        return F16
    if dt == np.float32:
        return F32
    raise ValueError(f"no EXL3 dtype code for {dt} (bf16 is passed as uint16 with code {BF16})")


# ---- thin numpy-facing wrappers over the C oracle ---------------------------------------------

def codebook_table(cb: int) -> np.ndarray:
    out = np.empty(65536, np.uint16)
    lib().exl3o_codebook_table(cb, _ptr(out))
    return out.view(np.float16)


def pack(states, k: int) -> np.ndarray:
    s = _u16(states).ravel()
    out = np.empty(s.size // 256 * 16 * k, np.uint16)
    if lib().exl3o_pack(_ptr(s), s.size, k, _ptr(out)):
        raise ValueError("pack: bad arguments")
    return out


def unpack(packed, k: int) -> np.ndarray:
    p = _u16(packed).ravel()
    out = np.empty(p.size // (16 * k) * 256, np.uint16)
    if lib().exl3o_unpack(_ptr(p), p.size, k, _ptr(out)):
        raise ValueError("unpack: bad arguments")
    return out


def permutation() -> np.ndarray:
    out = np.empty(256, np.int32)
    lib().exl3o_permutation(_ptr(out))
    return out


def permutation_inverse() -> np.ndarray:
    out = np.empty(256, np.int32)
    lib().exl3o_permutation_inverse(_ptr(out))
    return out


def reconstruct_inner(trellis, k: int, cb: int, threads: int | None = None) -> np.ndarray:
    """trellis [in/16, out/16, 16k] u16 -> W [in, out] fp16."""
    t = _u16(trellis)
    rows, cols = t.shape[0] * 16, t.shape[1] * 16
    out = np.empty((rows, cols), np.uint16)
    if lib().exl3o_reconstruct_inner(_ptr(t), k, cb, rows, cols, _ptr(out), threads or default_threads()):
        raise ValueError("reconstruct_inner: bad arguments")
    return out.view(np.float16)


def hadamard128(x) -> np.ndarray:
    """fp16 [..., 128*n] -> fp16, the transform MLX applies to fp16 data (scale 2^-3.5 included)."""
    a = _u16(x)
    out = np.empty_like(a)
    lib().exl3o_hadamard128(_ptr(a), _ptr(out), a.size // 128)
    return out.view(np.float16)


def prepare(x: np.ndarray, suh, x_dtype: int | None = None) -> np.ndarray:
    """x [rows, in] (f16/f32, or bf16 bits with x_dtype=BF16), suh [in] or [rows, in] -> xhat fp16."""
    code = x_dtype if x_dtype is not None else dtype_code(x.dtype)
    x = np.ascontiguousarray(x)
    rows, n = x.shape
    s = _u16(suh)
    scale_rows = 1 if s.ndim == 1 else s.shape[0]
    out = np.empty((rows, n), np.uint16)
    if lib().exl3o_prepare(_ptr(x), code, _ptr(s), scale_rows, rows, n, _ptr(out)):
        raise ValueError("prepare: bad arguments")
    return out.view(np.float16)


def finish(yhat: np.ndarray, svh, bias=None, y_dtype: int = F16) -> np.ndarray:
    yhat = np.ascontiguousarray(yhat, np.float32)
    rows, n = yhat.shape
    s = _u16(svh)
    scale_rows = 1 if s.ndim == 1 else s.shape[0]
    b = None if bias is None else _u16(bias)
    out = np.empty((rows, n), np.float32 if y_dtype == F32 else np.uint16)
    if lib().exl3o_finish(_ptr(yhat), _ptr(s), scale_rows, _ptr(b), rows, n, y_dtype, _ptr(out)):
        raise ValueError("finish: bad arguments")
    return out if y_dtype != F16 else out.view(np.float16)


def matmul_raw(trellis, k: int, cb: int, xhat, tk_range=None, f64acc: bool = False,
               threads: int | None = None) -> np.ndarray:
    """fp32 yhat [rows, out] = xhat [rows, in] fp16 times the decoded inner matrix."""
    t = _u16(trellis)
    n_in, n_out = t.shape[0] * 16, t.shape[1] * 16
    xh = _u16(xhat)
    rows = xh.shape[0]
    lo, hi = tk_range if tk_range is not None else (0, n_in // 16)
    out = np.empty((rows, n_out), np.float32)
    if lib().exl3o_matmul_raw(_ptr(t), k, cb, n_in, n_out, _ptr(xh), rows, lo, hi, int(f64acc), _ptr(out),
                              threads or default_threads()):
        raise ValueError("matmul_raw: bad arguments")
    return out


def linear_forward(trellis, k: int, cb: int, suh, svh, bias, x: np.ndarray, x_dtype: int | None = None,
                   threads: int | None = None) -> np.ndarray:
    """Exl3Linear.forward on the CPU: x [rows, in] -> y [rows, out] in x's dtype."""
    code = x_dtype if x_dtype is not None else dtype_code(x.dtype)
    t = _u16(trellis)
    n_in, n_out = t.shape[0] * 16, t.shape[1] * 16
    x = np.ascontiguousarray(x)
    rows = x.shape[0]
    b = None if bias is None else _u16(bias)
    out = np.empty((rows, n_out), np.float32 if code == F32 else np.uint16)
    s_in, s_out = _u16(suh), _u16(svh)
    if lib().exl3o_linear_forward(_ptr(t), k, cb, n_in, n_out, _ptr(s_in), _ptr(s_out), _ptr(b), _ptr(x), code,
                                  rows, _ptr(out), threads or default_threads()):
        raise ValueError("linear_forward: bad arguments")
    return out.view(np.float16) if code == F16 else out


def glu_down_input(gate_raw, up_raw, svh_gate, svh_up, down_suh) -> np.ndarray:
    g = np.ascontiguousarray(gate_raw, np.float32)
    u = np.ascontiguousarray(up_raw, np.float32)
    routes, h = g.shape
    a, b, c = _u16(svh_gate), _u16(svh_up), _u16(down_suh)
    out = np.empty((routes, h), np.uint16)
    if lib().exl3o_glu_down_input(_ptr(g), _ptr(u), _ptr(a), _ptr(b), _ptr(c), routes, h, _ptr(out)):
        raise ValueError("glu_down_input: bad arguments")
    return out.view(np.float16)


def finish_and_reduce(down_raw, down_svh, scores, top_k: int) -> np.ndarray:
    d = np.ascontiguousarray(down_raw, np.float32)
    routes, n = d.shape
    s, w = _u16(down_svh), _u16(scores).ravel()
    rows = routes // top_k
    out = np.empty((rows, n), np.uint16)
    if lib().exl3o_finish_and_reduce(_ptr(d), _ptr(s), _ptr(w), rows, top_k, n, _ptr(out)):
        raise ValueError("finish_and_reduce: bad arguments")
    return out.view(np.float16)


def switch_glu_forward(gu_trellis, gu_suh, gu_svh, down_trellis, down_suh, down_svh, top_k: int, k: int, cb: int,
                       x: np.ndarray, selected, scores, x_dtype: int | None = None) -> np.ndarray:
    """``Exl3SwitchGlu::forward`` for SiLU models (native/src/moe.rs:905-971), one slot at a time: routed input
    rotation (moe.rs:184-236), gate and up products on the expert's columns of the bank (gate columns of all
    experts, then up columns: native/src/linear.rs:2817-2885), ``glu_down_input``, down product,
    ``finish_and_reduce``.  ``scores`` fp16; result fp16 ``[rows, in]``."""
    gu_t, down_t = _u16(gu_trellis), _u16(down_trellis)
    gu_suh, gu_svh = np.asarray(gu_suh, np.float16), np.asarray(gu_svh, np.float16)
    down_suh, down_svh = np.asarray(down_suh, np.float16), np.asarray(down_svh, np.float16)
    experts, _, n_in = gu_suh.shape
    hidden = gu_svh.shape[2]
    sel = np.asarray(selected).reshape(-1)
    rows = x.shape[0]
    ht, it = hidden // 16, n_in // 16
    down_raw = np.empty((rows * top_k, n_in), np.float32)
    for slot, e in enumerate(sel):
        e = int(e)
        xr = x[slot // top_k: slot // top_k + 1]
        raw = []
        for p in range(2):
            xhat = prepare(xr, gu_suh[e, p], x_dtype)
            c0 = p * experts * ht + e * ht
            raw.append(matmul_raw(np.ascontiguousarray(gu_t[:, c0:c0 + ht]), k, cb, xhat))
        xd = glu_down_input(raw[0], raw[1], gu_svh[e, 0][None], gu_svh[e, 1][None], down_suh[e][None])
        down_raw[slot] = matmul_raw(np.ascontiguousarray(down_t[:, e * it:(e + 1) * it]), k, cb, xd)[0]
    return finish_and_reduce(down_raw, down_svh[sel], np.asarray(scores, np.float16), top_k)
