"""B200-native EXL3 quantized-linear path: hand-written sm_100a CUDA kernels behind a C ABI
(``include/b200exl3.h``), with this package as the Python host-side mirror of the reference's
operator interface.  Importing the package does not load the CUDA library; the first call does,
and it raises if the library is not built -- there is no CPU fallback.
"""
from ._lib import BF16, F16, F32, B200Exl3Error, LIB_PATH
from .linear import DEFAULT, MCG, MUL1, Exl3Group, Exl3Linear, Prologue, new_workspace, static_status, workspace_status
from .moe import Exl3SwitchGlu
from .stack import Exl3Stack
from .runtime import DEFAULT_STREAM, DeviceBuffer, Event, Graph, PinnedBuffer, Stream, init, set_option
from . import checkpoint, codec, decoder, ep, router

__all__ = [
    "BF16", "F16", "F32", "B200Exl3Error", "LIB_PATH", "DEFAULT", "MCG", "MUL1", "Exl3Group", "Exl3Linear", "Prologue", "new_workspace", "static_status", "workspace_status", "DEFAULT_STREAM",
    "Exl3SwitchGlu", "Exl3Stack", "DeviceBuffer", "Event", "Graph", "PinnedBuffer", "Stream", "init", "set_option", "checkpoint", "codec", "decoder", "ep", "router",
]
