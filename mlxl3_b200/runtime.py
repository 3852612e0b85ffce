"""Device plumbing over the C ABI: device and pinned buffers, streams and events.

The library owns no tensor type; these small wrappers exist so that Python hosts (tests, the
benchmark, the operator mirror in :mod:`mlxl3_b200.linear`) can move bytes without PyTorch.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_void_p

import numpy as np

from . import _lib

_initialised: set[int] = set()


def init(device: int = 0) -> None:
    """Selects the device for this thread (``b200exl3_init``).  Raises if it is not a B200-class GPU."""
    _lib.call("b200exl3_init", device)
    _initialised.add(device)


def set_option(name: str, value: int) -> None:
    _lib.call("b200exl3_set_option", name.encode(), int(value))


class Stream:
    def __init__(self, handle: int | None = None):
        self._own = handle is None
        if handle is None:
            h = c_void_p()
            _lib.call("b200exl3_stream_create", byref(h))
            handle = h.value
        self.handle = handle

    def sync(self) -> None:
        _lib.call("b200exl3_stream_sync", c_void_p(self.handle))

    def close(self) -> None:
        if self._own and self.handle:
            _lib.call("b200exl3_stream_destroy", c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


DEFAULT_STREAM = Stream(handle=0)


class Event:
    def __init__(self):
        h = c_void_p()
        _lib.call("b200exl3_event_create", byref(h))
        self.handle = h.value

    def record(self, stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_event_record", c_void_p(self.handle), c_void_p(stream.handle))

    def elapsed_ms(self, stop: "Event") -> float:
        """Milliseconds from this event to ``stop`` (waits for ``stop``)."""
        out = c_float()
        _lib.call("b200exl3_event_elapsed_ms", c_void_p(self.handle), c_void_p(stop.handle), byref(out))
        return out.value

    def __del__(self):
        try:
            if self.handle:
                _lib.call("b200exl3_event_destroy", c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass


class DeviceBuffer:
    """``nbytes`` of device memory owned through ``b200exl3_malloc`` / ``b200exl3_free``."""

    def __init__(self, nbytes: int):
        p = c_void_p()
        _lib.call("b200exl3_malloc", int(nbytes), byref(p))
        self.ptr = p.value or 0
        self.nbytes = int(nbytes)

    @classmethod
    def from_numpy(cls, array: np.ndarray, stream: Stream = DEFAULT_STREAM) -> "DeviceBuffer":
        a = np.ascontiguousarray(array)
        buf = cls(a.nbytes)
        buf.upload(a, stream)
        stream.sync()
        return buf

    def upload(self, array: np.ndarray, stream: Stream = DEFAULT_STREAM, offset: int = 0) -> None:
        a = np.ascontiguousarray(array)
        if offset + a.nbytes > self.nbytes:
            raise ValueError("upload exceeds the device buffer")
        _lib.call("b200exl3_memcpy_h2d", c_void_p(self.ptr + offset), a.ctypes.data_as(c_void_p), a.nbytes,
                  c_void_p(stream.handle))

    def download(self, shape, dtype, stream: Stream = DEFAULT_STREAM, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype)
        if offset + out.nbytes > self.nbytes:
            raise ValueError("download exceeds the device buffer")
        _lib.call("b200exl3_memcpy_d2h", out.ctypes.data_as(c_void_p), c_void_p(self.ptr + offset), out.nbytes,
                  c_void_p(stream.handle))
        stream.sync()
        return out

    def fill(self, byte: int, stream: Stream = DEFAULT_STREAM) -> None:
        _lib.call("b200exl3_memset", c_void_p(self.ptr), byte, self.nbytes, c_void_p(stream.handle))

    def free(self) -> None:
        if self.ptr:
            _lib.call("b200exl3_free", c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PinnedBuffer:
    """Page-locked host memory exposed as a numpy array, for timed host<->device copies."""

    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        p = c_void_p()
        _lib.call("b200exl3_host_alloc", max(self.nbytes, 1), byref(p))
        self.ptr = p.value
        raw = (ctypes.c_char * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            _lib.call("b200exl3_host_free", c_void_p(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Graph:
    """A recorded sequence of launches (``b200exl3_graph_*``), replayed with one call.

    with Graph.record(stream) as g:
        ... forward_device calls on `stream` ...
    g.launch(stream)
    """

    def __init__(self):
        self.handle = None
        self._stream = None

    @classmethod
    def record(cls, stream: Stream) -> "Graph":
        g = cls()
        g._stream = stream
        return g

    def __enter__(self) -> "Graph":
        _lib.call("b200exl3_graph_begin", c_void_p(self._stream.handle))
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        h = c_void_p()
        status = _lib.load().b200exl3_graph_end(c_void_p(self._stream.handle), byref(h))
        if exc_type is None:
            _lib.check(status)
            self.handle = h.value

    def launch(self, stream: Stream) -> None:
        _lib.call("b200exl3_graph_launch", c_void_p(self.handle), c_void_p(stream.handle))

    def __del__(self):
        try:
            if self.handle:
                _lib.call("b200exl3_graph_free", c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass
