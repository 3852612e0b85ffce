"""Shared helpers of the GPU parity tests."""
import numpy as np
import pytest


@pytest.fixture(scope="session")
def gpu():
    import mlxl3_b200
    mlxl3_b200.init(0)          # raises unless device 0 is an sm_100 GPU and the CUDA library is built
    return mlxl3_b200


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint16)


def random_layer(rng, n_in, n_out, k, signs=True):
    trellis = rng.integers(0, 65536, (n_in // 16, n_out // 16, 16 * k), dtype=np.uint16)
    if signs:
        suh = np.where(rng.random(n_in) > 0.5, -1, 1).astype(np.float16)
        svh = np.where(rng.random(n_out) > 0.5, -1, 1).astype(np.float16)
    else:
        suh = rng.uniform(0.5, 1.5, n_in).astype(np.float16)
        svh = rng.uniform(0.5, 1.5, n_out).astype(np.float16)
    return trellis, suh, svh


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)
