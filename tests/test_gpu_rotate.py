"""GPU parity of the Hadamard-128 rotations, through the C ABI: bit-identical to the oracle and to the
reference's SHA-256 known answers."""
import hashlib
import json

import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, from_bf16_bits, gpu, to_bf16_bits  # noqa: F401
from tests.test_oracle_golden import _h128_cases

pytestmark = pytest.mark.gpu


def test_h128_known_answers(gpu, golden_dir):
    kat = json.loads((golden_dir / "h128_kat.json").read_text())["cases"]
    seen = set()
    for name, x, scales in _h128_cases():
        s = scales[0] if scales.shape[0] == 1 else scales
        got = gpu.codec.prepare(x, s)
        assert got.size == kat[name]["values"]
        assert hashlib.sha256(bits(got).astype("<u2").tobytes()).hexdigest() == kat[name]["f16le_sha256"], name
        seen.add(name)
    assert seen == set(kat)


@pytest.mark.parametrize("rows,width", [(1, 128), (5, 4096), (33, 384), (512, 1024)])
def test_prepare_dtypes(gpu, rows, width):
    rng = np.random.default_rng(rows * 7 + width)
    suh = rng.uniform(0.5, 1.5, width).astype(np.float16)
    x32 = (rng.standard_normal((rows, width)) * 3).astype(np.float32)
    for x, code in ((x32.astype(np.float16), None), (x32, None)):
        assert np.array_equal(bits(gpu.codec.prepare(x, suh, code)), bits(oracle.prepare(x, suh)))
    xb = to_bf16_bits(x32)
    want = oracle.prepare(xb, suh, x_dtype=oracle.BF16)
    assert np.array_equal(bits(gpu.codec.prepare(xb, suh, gpu.BF16)), bits(want))
    per_row = rng.uniform(0.5, 1.5, (rows, width)).astype(np.float16)
    assert np.array_equal(bits(gpu.codec.prepare(x32, per_row)), bits(oracle.prepare(x32, per_row)))


@pytest.mark.parametrize("rows,width,splits", [(1, 128, 1), (3, 4096, 2), (17, 256, 5)])
def test_finish(gpu, rows, width, splits):
    rng = np.random.default_rng(rows + width + splits)
    partials = (rng.standard_normal((splits, rows, width)) * 30).astype(np.float32)
    svh = rng.uniform(0.5, 1.5, width).astype(np.float16)
    bias = (rng.standard_normal(width) * 0.2).astype(np.float16)
    total = partials[0].copy()
    for s in range(1, splits):
        total = total + partials[s]                                    # fp32, in split order
    for b in (None, bias):
        got = gpu.codec.finish(partials, svh, b)
        assert np.array_equal(bits(got), bits(oracle.finish(total, svh, b)))
        got32 = gpu.codec.finish(partials, svh, b, y_dtype=gpu.F32)
        assert np.array_equal(got32, oracle.finish(total, svh, b, y_dtype=oracle.F32))
        gotb = gpu.codec.finish(partials, svh, b, y_dtype=gpu.BF16)
        assert np.array_equal(gotb, oracle.finish(total, svh, b, y_dtype=oracle.BF16))


def test_rotation_edge_cases(gpu):
    assert gpu.codec.prepare(np.empty((0, 128), np.float16), np.ones(128, np.float16)).shape == (0, 128)
    with pytest.raises(gpu.B200Exl3Error, match="128-aligned"):
        gpu.codec.prepare(np.zeros((1, 127), np.float16), np.ones(127, np.float16))
    # an involution up to rounding: H128(H128(x)) == x for exactly representable inputs
    x = np.zeros((1, 128), np.float16)
    x[0, 5] = 8.0
    once = gpu.codec.prepare(x, np.ones(128, np.float16))
    twice = gpu.codec.prepare(once, np.ones(128, np.float16))
    assert np.allclose(twice.astype(np.float32), x.astype(np.float32), atol=2e-3)
