"""CPU-only checks of the C-ABI library: it loads, exports every declared symbol, and fails loudly."""
import ctypes
import re

import numpy as np
import pytest

import mlxl3_b200
from mlxl3_b200 import _lib
from tests.conftest import ROOT


def test_every_declared_symbol_is_exported_and_bound():
    header = (ROOT / "include" / "b200exl3.h").read_text()
    declared = set(re.findall(r"\b(b200exl3_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES)


def test_library_has_no_torch_dependency():
    import subprocess
    out = subprocess.run(["ldd", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    names = [line.split()[0] for line in out.splitlines() if line.strip()]          # library names only, not load addresses
    assert names and not any("torch" in n or "c10" in n for n in names)


def test_version_and_error_string_without_a_gpu():
    lib = _lib.load()
    assert lib.b200exl3_version() >= 100
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device error path cannot be exercised")
    with pytest.raises(_lib.B200Exl3Error) as err:
        mlxl3_b200.init(0)
    assert "cuda" in str(err.value).lower()
    assert lib.b200exl3_set_option(b"no_such_option", 1) == -1
    assert b"unknown option" in lib.b200exl3_last_error()
    # argument validation happens before any CUDA call
    out = ctypes.c_void_p()
    assert lib.b200exl3_linear_create(None, None, None, None, 9, 128, 128, 9, 0, 0, ctypes.byref(out)) == -1
    assert b"K must be in 1..=8" in lib.b200exl3_last_error()
    assert lib.b200exl3_linear_create(None, None, None, None, 9, 100, 128, 4, 0, 0, ctypes.byref(out)) == -1
    assert b"128-aligned" in lib.b200exl3_last_error()
    assert lib.b200exl3_linear_create(None, None, None, None, 9, 128, 128, 4, 3, 0, ctypes.byref(out)) == -1
    assert b"invalid EXL3 codebook 3" in lib.b200exl3_last_error()
    assert lib.b200exl3_prepare(None, 9, None, 1, 1, 127, None, None) == -1
    assert b"expected complete 128-aligned rows" in lib.b200exl3_last_error()


@pytest.mark.parametrize("kwargs,message", [
    (dict(k=9), "K must be in 1..=8"),
    (dict(cb=3), "invalid EXL3 codebook"),
    (dict(trellis_shape=(8, 8, 48)), "invalid trellis shape"),
    (dict(trellis_shape=(8, 7, 64)), "128-aligned"),
    (dict(suh_len=127), "scales have wrong dimensions"),
    (dict(bias_len=5), "bias has wrong dimensions"),
    (dict(trellis_dtype=np.int32), "16-bit integers"),
])
def test_operator_validation_matches_reference_wording(kwargs, message):
    # native/src/linear.rs:577-639 of the reference
    k = kwargs.get("k", 4)
    shape = kwargs.get("trellis_shape", (8, 8, 16 * min(k, 8)))
    trellis = np.zeros(shape, kwargs.get("trellis_dtype", np.uint16))
    suh = np.ones(kwargs.get("suh_len", shape[0] * 16), np.float16)
    svh = np.ones(shape[1] * 16, np.float16)
    bias = np.ones(kwargs["bias_len"], np.float16) if "bias_len" in kwargs else None
    with pytest.raises(mlxl3_b200.B200Exl3Error) as err:
        mlxl3_b200.Exl3Linear(trellis, suh, svh, bias, k, kwargs.get("cb", 0))
    assert message in str(err.value)
