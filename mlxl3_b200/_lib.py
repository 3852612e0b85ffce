"""ctypes binding of ``libb200exl3.so``: one Python declaration per symbol of ``include/b200exl3.h``.

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200exl3.so"

U16, U32, F16, F32, BF16 = 2, 3, 9, 10, 12
EXACT_WEIGHTS = 2
WORKSPACE_HEADER_BYTES = 16384


class B200Exl3Error(RuntimeError):
    """An entry point of the C ABI returned -1; the message is the library's thread-local error string."""


# name -> (restype, argtypes); must list every symbol the header declares (a CPU test checks this).
SIGNATURES = {
    "b200exl3_init": (c_int, [c_int]),
    "b200exl3_last_error": (c_char_p, []),
    "b200exl3_version": (c_int, []),
    "b200exl3_set_option": (c_int, [c_char_p, c_int64]),
    "b200exl3_plan_query": (c_int, [c_char_p, c_int, c_int, c_int, c_int64, POINTER(c_int64), c_int]),
    "b200exl3_malloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "b200exl3_free": (c_int, [c_void_p]),
    "b200exl3_host_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "b200exl3_host_free": (c_int, [c_void_p]),
    "b200exl3_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
    "b200exl3_stream_create": (c_int, [POINTER(c_void_p)]),
    "b200exl3_stream_destroy": (c_int, [c_void_p]),
    "b200exl3_stream_sync": (c_int, [c_void_p]),
    "b200exl3_event_create": (c_int, [POINTER(c_void_p)]),
    "b200exl3_event_destroy": (c_int, [c_void_p]),
    "b200exl3_event_record": (c_int, [c_void_p, c_void_p]),
    "b200exl3_event_elapsed_ms": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
    "b200exl3_graph_begin": (c_int, [c_void_p]),
    "b200exl3_graph_end": (c_int, [c_void_p, POINTER(c_void_p)]),
    "b200exl3_graph_launch": (c_int, [c_void_p, c_void_p]),
    "b200exl3_graph_free": (c_int, [c_void_p]),
    "b200exl3_unpack_states": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200exl3_codebook": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_reconstruct": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200exl3_prepare": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_finish": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200exl3_linear_create": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                       c_uint32, POINTER(c_void_p)]),
    "b200exl3_linear_free": (None, [c_void_p]),
    "b200exl3_linear_input_dims": (c_int, [c_void_p]),
    "b200exl3_linear_output_dims": (c_int, [c_void_p]),
    "b200exl3_linear_workspace_bytes": (c_int, [c_void_p, c_int64, POINTER(c_size_t)]),
    "b200exl3_workspace_status": (c_int, [c_void_p, POINTER(c_int)]),
    "b200exl3_linear_forward": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_linear_forward_static": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "b200exl3_static_status": (c_int, [POINTER(c_int), c_int]),
    "b200exl3_linear_forward_raw": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_linear_forward_partial": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_size_t,
                                                c_void_p]),
    "b200exl3_linear_finish": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_linear_decode": (c_int, [c_void_p, c_void_p, c_void_p]),
    "b200exl3_group_create": (c_int, [POINTER(c_void_p), c_int, POINTER(c_void_p)]),
    "b200exl3_group_free": (None, [c_void_p]),
    "b200exl3_group_count": (c_int, [c_void_p]),
    "b200exl3_group_workspace_bytes": (c_int, [c_void_p, c_int64, POINTER(c_size_t)]),
    "b200exl3_group_forward": (c_int, [c_void_p, c_void_p, c_int, c_int64, POINTER(c_void_p), c_void_p, c_size_t, c_void_p]),
    "b200exl3_linear_forward_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_group_forward_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, POINTER(c_void_p), c_void_p, c_size_t, c_void_p]),
    "b200exl3_stack_create": (c_int, [c_void_p, c_int, c_int, c_int64, POINTER(c_void_p)]),
    "b200exl3_stack_free": (None, [c_void_p]),
    "b200exl3_stack_forward": (c_int, [c_void_p, c_void_p]),
    "b200exl3_stack_status": (c_int, [c_void_p, POINTER(c_int)]),
    "b200exl3_stack_reset": (c_int, [c_void_p]),
    "b200exl3_stack_geometry": (c_int, [c_void_p, POINTER(c_int), POINTER(c_size_t)]),
    "b200exl3_expert_mapped": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64,
                                       c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200exl3_swiglu_down_input": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_finish_and_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200exl3_ipc_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_char_p]),
    "b200exl3_ep_buffer_bytes": (c_int, [c_int, c_int, POINTER(c_size_t)]),
    "b200exl3_ep_create": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_void_p), POINTER(c_void_p)]),
    "b200exl3_ep_free": (None, [c_void_p]),
    "b200exl3_ep_status": (c_int, [c_void_p, POINTER(c_int)]),
    "b200exl3_moe_ep_workspace_bytes": (c_int, [c_void_p, c_int64, POINTER(c_size_t)]),
    "b200exl3_moe_forward_ep": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_size_t, c_void_p]),
    "b200exl3_embed": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "b200exl3_swiglu": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200exl3_rope_append": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "b200exl3_attention_workspace_bytes": (c_int, [c_int, c_int, POINTER(c_size_t)]),
    "b200exl3_attention_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_head_workspace_bytes": (c_int, [POINTER(c_size_t)]),
    "b200exl3_head_argmax": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_router_topk": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200exl3_router_softmax_topk": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200exl3_router_gate": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200exl3_tp_buffer_bytes": (c_int, [c_int, c_int, POINTER(c_size_t)]),
    "b200exl3_tp_alloc": (c_int, [c_int, c_int, POINTER(c_void_p), c_char_p]),
    "b200exl3_tp_open": (c_int, [c_char_p, POINTER(c_void_p)]),
    "b200exl3_tp_close": (c_int, [c_void_p]),
    "b200exl3_tp_create": (c_int, [c_int, c_int, c_int, POINTER(c_void_p), POINTER(c_void_p)]),
    "b200exl3_tp_free": (None, [c_void_p]),
    "b200exl3_tp_status": (c_int, [c_void_p, POINTER(c_int)]),
    "b200exl3_tp_reset": (c_int, [c_void_p]),
    "b200exl3_linear_forward_tp": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200exl3_linear_finish_tp": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "b200exl3_moe_create": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_uint32, POINTER(c_void_p)]),
    "b200exl3_moe_free": (None, [c_void_p]),
    "b200exl3_moe_workspace_bytes": (c_int, [c_void_p, c_int64, POINTER(c_size_t)]),
    "b200exl3_moe_forward": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_size_t, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and declares every signature.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise B200Exl3Error(
            f"{LIB_PATH} is missing: build it with `python -m mlxl3_b200.build` (there is no CPU fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise B200Exl3Error(load().b200exl3_last_error().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))
