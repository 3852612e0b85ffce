"""JSON-lines codec tool, wire-compatible with the reference's ``mlxl3-rs codec`` (native/src/main.rs:286-427,
540-676, 1350-1368): one JSON object per input line, one ``{"data": ...}`` or ``{"error": "..."}`` per output
line; a bad request does not end the loop.  Lets the reference's differential drivers
(native/check_qmm_tiles.py) talk to this implementation op for op.

    python -m mlxl3_b200.codec_cli < requests.jsonl > responses.jsonl

Operations: ``pack``, ``unpack``, ``codebook``, ``permutation`` (format), ``mlx-linear``, ``mlx-group``,
``mlx-switch`` (operators; 16-bit arrays travel as integer bit patterns).  Common fields: ``op``, ``k`` (default
4), ``mode`` (codebook 0/1/2), ``data`` (uint16 array).
"""
from __future__ import annotations

import json
import sys

import numpy as np

from . import B200Exl3Error, Exl3Group, Exl3Linear, Exl3SwitchGlu, codec, init


def _u16(request: dict, key: str) -> np.ndarray:
    return np.asarray(request.get(key, []), dtype=np.uint16)


def _f16(request: dict, key: str, shape) -> np.ndarray:
    return _u16(request, key).view(np.float16).reshape(shape)


def _check_k(k: int) -> None:
    if not 1 <= k <= 8:
        raise B200Exl3Error(f"K must be in 1..=8, got {k}")


def _linear(request: dict, k: int, cb: int):
    _check_k(k)
    rows = len(request.get("suh", []))
    x = _u16(request, "x")
    if rows <= 0 or x.size % rows:
        raise B200Exl3Error("invalid linear input rows")
    cols = int(request.get("cols", 0))
    trellis = _u16(request, "data").reshape(rows // 16, cols // 16, 16 * k)
    layer = Exl3Linear(trellis, _f16(request, "suh", (rows,)), _f16(request, "svh", (cols,)), None, k, cb,
                       exact_weights=True)
    try:
        return layer.forward(x.view(np.float16).reshape(-1, rows)).view(np.uint16).reshape(-1).tolist()
    finally:
        layer.close()


def _group(request: dict, k: int, cb: int):
    _check_k(k)
    widths = [int(w) for w in request.get("widths", [])]
    suh, svh, data, x = (_u16(request, key) for key in ("suh", "svh", "data", "x"))
    if not widths:
        raise B200Exl3Error("missing group widths")
    if suh.size % len(widths):
        raise B200Exl3Error("invalid grouped input scales")
    rows = suh.size // len(widths)
    if rows <= 0 or rows % 128 or x.size % rows:
        raise B200Exl3Error("invalid grouped input size")
    if len(widths) < 2 or k == 7:
        raise B200Exl3Error("unsupported group")
    members, at, scale_at = [], 0, 0
    try:
        for index, width in enumerate(widths):
            if width <= 0 or width % 128:
                raise B200Exl3Error("invalid group width")
            words = (rows // 16) * (width // 16) * 16 * k
            if at + words > data.size:
                raise B200Exl3Error("truncated grouped trellis")
            if scale_at + width > svh.size:
                raise B200Exl3Error("truncated grouped scales")
            members.append(Exl3Linear(data[at:at + words].reshape(rows // 16, width // 16, 16 * k),
                                      suh[index * rows:(index + 1) * rows].view(np.float16),
                                      svh[scale_at:scale_at + width].view(np.float16), None, k, cb, exact_weights=True))
            at += words
            scale_at += width
        if at != data.size or scale_at != svh.size:
            raise B200Exl3Error("extra grouped data")
        group = Exl3Group(members)
        try:
            outputs = group.forward(x.view(np.float16).reshape(-1, rows))
            return [y.view(np.uint16).reshape(-1).tolist() for y in outputs]
        finally:
            group.close()
    finally:
        for member in members:
            member.close()


def _switch(request: dict, k: int, cb: int):
    experts = int(request.get("key_heads", 0))
    selected = np.asarray(request.get("selected", []), dtype=np.uint32)
    top_k = int(request.get("top_k", 0)) or selected.size
    if top_k <= 0 or selected.size % top_k:
        raise B200Exl3Error("invalid SwitchGLU routes")
    rows = selected.size // top_k
    x = _u16(request, "x")
    if rows <= 0 or x.size % rows:
        raise B200Exl3Error("invalid SwitchGLU rows")
    n_in, hidden = x.size // rows, int(request.get("cols", 0))
    block = Exl3SwitchGlu(_u16(request, "data").reshape(n_in // 16, experts * hidden // 8, 16 * k),
                          _f16(request, "suh", (experts, 2, n_in)), _f16(request, "svh", (experts, 2, hidden)),
                          _u16(request, "down_data").reshape(hidden // 16, experts * n_in // 16, 16 * k),
                          _f16(request, "down_suh", (experts, hidden)), _f16(request, "down_svh", (experts, n_in)),
                          top_k, k, cb, exact_weights=True)
    try:
        y = block.forward(x.view(np.float16).reshape(rows, n_in), selected.reshape(rows, top_k),
                          _f16(request, "beta", (rows, top_k)))
        return y.view(np.uint16).reshape(-1).tolist()
    finally:
        block.close()


def _expert(request: dict, k: int, cb: int):
    """``mlx-expert`` (native/src/main.rs:540-597): field for field."""
    from .moe import expert_mapped
    projections = int(request.get("projections_per_route", 0))
    selected = np.asarray(request.get("selected", []), dtype=np.uint32)
    if projections <= 0:
        raise B200Exl3Error("invalid projection count")
    rows = selected.size * projections
    if rows <= 0:
        raise B200Exl3Error("missing expert routes")
    x = _u16(request, "x")
    if x.size % rows:
        raise B200Exl3Error("invalid expert input dimensions")
    n_in, cols = x.size // rows, int(request.get("cols", 0))
    data = _u16(request, "data")
    per_column = (n_in // 16) * 16 * k
    if n_in <= 0 or n_in % 16 or data.size % per_column:
        raise B200Exl3Error("invalid expert trellis dimensions")
    raw = bool(request.get("return_raw", False))
    out = expert_mapped(x.view(np.float16).reshape(rows, n_in), data.reshape(n_in // 16, data.size // per_column, 16 * k),
                        _f16(request, "suh", (rows, n_in)), None if raw else _f16(request, "svh", (rows, cols)), selected, cols, projections,
                        int(request.get("projection_stride_tiles", 0)), k, cb, False, raw)
    return {"f32": out.reshape(-1).tolist()} if raw else {"f16": out.view(np.uint16).reshape(-1).tolist()}


def _swiglu_prepare(request: dict):
    """``mlx-swiglu-prepare`` (native/src/main.rs:599-614): ``suh`` carries the gate/up output scales [experts, 2, hidden],
    ``svh`` the down input scales [experts, hidden]."""
    from .moe import swiglu_down_input
    hidden = int(request.get("cols", 0))
    selected = np.asarray(request.get("selected", []), dtype=np.uint32)
    scales = _u16(request, "suh")
    if hidden <= 0 or scales.size % (2 * hidden):
        raise B200Exl3Error("invalid gate/up scales")
    experts = scales.size // (2 * hidden)
    state = np.asarray(request.get("state", []), dtype=np.float32).reshape(selected.size * 2, hidden)
    out = swiglu_down_input(state, scales.view(np.float16).reshape(experts, 2, hidden), _f16(request, "svh", (experts, hidden)), selected)
    return out.view(np.uint16).reshape(-1).tolist()


def _expert_reduce(request: dict):
    """``mlx-expert-reduce`` (native/src/main.rs:615-626): one output row from ``len(beta)`` slots."""
    from .moe import finish_and_reduce
    width = int(request.get("cols", 0))
    beta = _u16(request, "beta")
    slots = beta.size
    if width <= 0 or slots <= 0:
        raise B200Exl3Error("invalid expert reduction input")
    state = np.asarray(request.get("state", []), dtype=np.float32).reshape(slots, width)
    out = finish_and_reduce(state, _f16(request, "svh", (slots, width)), beta.view(np.float16).reshape(1, slots))
    return out.view(np.uint16).reshape(-1).tolist()


def handle(request: dict):
    """One request -> the value of its ``data`` answer (raises on a bad request)."""
    if not isinstance(request, dict) or not isinstance(request.get("op"), str):
        raise B200Exl3Error("invalid codec request")
    op, k, cb = request["op"], int(request.get("k", 4)), int(request.get("mode", 0))
    if cb not in (0, 1, 2):
        raise B200Exl3Error(f"invalid EXL3 codebook {cb}")
    if op == "pack":
        return codec.pack(_u16(request, "data"), k).tolist()
    if op == "unpack":
        return codec.unpack(_u16(request, "data"), k).reshape(-1).tolist()
    if op == "codebook":
        return codec.codebook(_u16(request, "data"), cb).view(np.uint16).reshape(-1).tolist()
    if op == "permutation":
        return codec.permutation().tolist()
    if op == "mlx-linear":
        return _linear(request, k, cb)
    if op == "mlx-group":
        return _group(request, k, cb)
    if op == "mlx-switch":
        return _switch(request, k, cb)
    if op == "mlx-expert":
        return _expert(request, k, cb)
    if op == "mlx-swiglu-prepare":
        return _swiglu_prepare(request)
    if op == "mlx-expert-reduce":
        return _expert_reduce(request)
    raise B200Exl3Error(f"unknown or unavailable codec operation {op}")


_DEVICE_OPS = ("unpack", "codebook", "mlx-linear", "mlx-group", "mlx-switch", "mlx-expert", "mlx-swiglu-prepare", "mlx-expert-reduce")


def main(stdin=None, stdout=None, device: int = 0) -> None:
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    ready = False
    for line in stdin:
        try:
            try:
                request = json.loads(line)
            except ValueError as error:
                raise B200Exl3Error("invalid codec request") from error
            if not ready and isinstance(request, dict) and request.get("op") in _DEVICE_OPS:
                init(device)                       # the GPU is only touched by operations that need it
                ready = True
            answer = {"data": handle(request)}
        except (B200Exl3Error, ValueError, TypeError, OverflowError) as error:
            answer = {"error": str(error)}
        stdout.write(json.dumps(answer, separators=(",", ":")) + "\n")
        stdout.flush()


if __name__ == "__main__":
    main()
