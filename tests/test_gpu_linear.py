"""GPU parity of Exl3Linear.forward (QMV and small-batch QMM) through the C ABI.

Tolerances.  The decoded weights and both rotations are bit-exact (tested elsewhere); the only
freedom is the fp32 accumulation order of the product and, in the default mode for codebooks 0/1,
feeding a weight as its two fp16 halves (x*lo + x*hi) instead of the fp16-rounded sum.  Stated bars:
  raw product  : max |got - f64| <= 2e-4 * max|f64| per row in exact mode, 1e-3 in split mode;
  layer output : max |got - oracle| <= 1e-2 * max|oracle| per row (the stated tolerance of the path),
                 and in exact mode an RMS difference below 1e-3 of the output RMS (what is left is the
                 fp32 summation order flipping the fp16 rounding of a few partial sums by one ulp).
"""
import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, from_bf16_bits, gpu, random_layer, to_bf16_bits  # noqa: F401

pytestmark = pytest.mark.gpu


def _check_raw(got, want64, rel):
    assert got.shape == want64.shape and np.isfinite(got).all()
    scale = np.abs(want64).max(axis=1, keepdims=True)
    assert (np.abs(got - want64) <= rel * scale).all(), float((np.abs(got - want64) / scale).max())


def _check_out(got, want, rel=1e-2):
    g, w = got.astype(np.float32), want.astype(np.float32)
    assert g.shape == w.shape and np.isfinite(g).all()
    scale = np.abs(w).max(axis=1, keepdims=True)
    assert (np.abs(g - w) <= rel * scale).all(), float((np.abs(g - w) / scale).max())


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", range(3))
def test_raw_product_all_formats(gpu, k, cb):
    rng = np.random.default_rng(1000 + 10 * k + cb)
    trellis, suh, svh = random_layer(rng, 256, 384, k)
    for exact in (True, False):
        layer = gpu.Exl3Linear(trellis, suh, svh, None, k, cb, exact_weights=exact)
        assert (layer.input_dims(), layer.output_dims()) == (256, 384)
        for rows in (1, 3, 8, 9, 16, 17, 32, 45):
            xhat = rng.standard_normal((rows, 256)).astype(np.float16)
            want = oracle.matmul_raw(trellis, k, cb, xhat, f64acc=True)
            _check_raw(layer.forward_raw(xhat), want, 2e-4 if exact or cb == 2 else 1e-3)
        layer.close()


@pytest.mark.parametrize("k,cb", [(4, 0), (3, 1), (2, 2), (6, 0), (8, 1), (5, 2), (1, 0), (7, 1)])
def test_forward_matches_oracle(gpu, k, cb):
    rng = np.random.default_rng(2000 + 10 * k + cb)
    trellis, suh, svh = random_layer(rng, 512, 256, k, signs=(k % 2 == 0))
    bias = (rng.standard_normal(256) * 0.1).astype(np.float16) if k % 3 == 0 else None
    exact = gpu.Exl3Linear(trellis, suh, svh, bias, k, cb, exact_weights=True)
    fast = gpu.Exl3Linear(trellis, suh, svh, bias, k, cb)
    inner = exact.decode()
    assert np.array_equal(bits(inner), bits(oracle.reconstruct_inner(trellis, k, cb)))
    for rows in (1, 2, 7, 16, 23, 40):
        x = rng.standard_normal((rows, 512)).astype(np.float16)
        want = oracle.linear_forward(trellis, k, cb, suh, svh, bias, x)
        got = exact.forward(x)
        assert got.dtype == np.float16
        _check_out(got, want)
        diff = got.astype(np.float32) - want.astype(np.float32)
        assert np.sqrt((diff ** 2).mean()) <= 1e-3 * np.sqrt((want.astype(np.float32) ** 2).mean())
        _check_out(fast.forward(x), want)
    # output dtype follows the input dtype (native/src/linear.rs:990-996 of the reference)
    x32 = rng.standard_normal((3, 512)).astype(np.float32)
    got32 = exact.forward(x32)
    assert got32.dtype == np.float32
    _check_out(got32, oracle.linear_forward(trellis, k, cb, suh, svh, bias, x32))
    xb = to_bf16_bits(x32)
    gotb = exact.forward(xb, dtype=gpu.BF16)
    wantb = oracle.linear_forward(trellis, k, cb, suh, svh, bias, xb, x_dtype=oracle.BF16)
    _check_out(from_bf16_bits(gotb), from_bf16_bits(wantb), rel=2e-2)
    # leading dimensions are kept
    x3 = rng.standard_normal((2, 3, 512)).astype(np.float16)
    assert exact.forward(x3).shape == (2, 3, 256)
    with pytest.raises(gpu.B200Exl3Error, match="invalid EXL3 linear input for 512 inputs"):
        exact.forward(np.zeros((1, 511), np.float16))
    with pytest.raises(gpu.B200Exl3Error, match="cannot be empty"):
        exact.forward(np.zeros((0, 512), np.float16))


@pytest.mark.parametrize("k,cb,rows", [(4, 0, 1), (3, 1, 5), (6, 2, 12), (8, 0, 16)])
def test_fused_rotations_are_bit_exact(gpu, k, cb, rows):
    # The fused kernel's input and output rotations must equal the oracle's bit for bit: feed the oracle's
    # rotated input to the raw product, rotate that product on the CPU, and compare with the fused call.
    rng = np.random.default_rng(300 + k)
    trellis, suh, svh = random_layer(rng, 1024, 384, k, signs=False)
    bias = (rng.standard_normal(384) * 0.3).astype(np.float16)
    layer = gpu.Exl3Linear(trellis, suh, svh, bias, k, cb)
    x = rng.standard_normal((rows, 1024)).astype(np.float16)
    gpu.set_option("qmm", 0)          # from 9 rows on a plain forward would take the tensor-core path: keep it on the fused kernel
    try:
        yhat = layer.forward_raw(oracle.prepare(x, suh))
        assert np.array_equal(bits(layer.forward(x)), bits(oracle.finish(yhat, svh, bias)))
        x32 = x.astype(np.float32) * 1.0009765625
        yhat32 = layer.forward_raw(oracle.prepare(x32, suh))
        assert np.array_equal(layer.forward(x32), oracle.finish(yhat32, svh, bias, y_dtype=oracle.F32))
    finally:
        gpu.set_option("qmm", 1)


def test_rows_are_independent_and_deterministic(gpu):
    # the reference checks batched rows against single rows byte for byte (native/src/linear.rs:3427-3430)
    rng = np.random.default_rng(77)
    trellis, suh, svh = random_layer(rng, 1024, 512, 4)
    layer = gpu.Exl3Linear(trellis, suh, svh, None, 4, 0)
    x = rng.standard_normal((8, 1024)).astype(np.float16)
    batched = layer.forward(x)
    assert np.array_equal(bits(batched), bits(layer.forward(x)))
    for r in range(8):
        assert np.array_equal(bits(layer.forward(x[r:r + 1])), bits(batched[r:r + 1]))


@pytest.mark.parametrize("grid", [1, 2, 3, 7, 64, 296, 1000])
def test_work_partition_does_not_change_parity(gpu, grid):
    # any number of CTAs: slices that span several column blocks, blocks shared by many CTAs
    rng = np.random.default_rng(5 + grid)
    trellis, suh, svh = random_layer(rng, 2048, 384, 4)
    gpu.set_option("qmv_force_grid", grid)
    try:
        layer = gpu.Exl3Linear(trellis, suh, svh, None, 4, 0, exact_weights=True)
        x = rng.standard_normal((5, 2048)).astype(np.float16)
        _check_out(layer.forward(x), oracle.linear_forward(trellis, 4, 0, suh, svh, None, x))
        xhat = oracle.prepare(x, suh)
        _check_raw(layer.forward_raw(xhat), oracle.matmul_raw(trellis, 4, 0, xhat, f64acc=True), 2e-4)
    finally:
        gpu.set_option("qmv_force_grid", 0)


@pytest.mark.parametrize("n_in,n_out,k,rows", [(4096, 4096, 4, 1), (4096, 14336, 3, 4), (14336, 4096, 3, 16)])
def test_full_size_layers(gpu, n_in, n_out, k, rows):
    # the single-layer configuration and the MLP-block shapes at small batch
    rng = np.random.default_rng(1001 if k == 4 else 2001)
    trellis, suh, svh = random_layer(rng, n_in, n_out, k)
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    want = oracle.linear_forward(trellis, k, 0, suh, svh, None, x)
    for exact in (True, False):
        layer = gpu.Exl3Linear(trellis, suh, svh, None, k, 0, exact_weights=exact)
        _check_out(layer.forward(x), want)
        layer.close()
    # linearity of the whole operator in x (size-independent property): f(2x) == 2 f(x) exactly in fp16
    layer = gpu.Exl3Linear(trellis, suh, svh, None, k, 0, exact_weights=True)
    y1, y2 = layer.forward(x), layer.forward((x * 2).astype(np.float16))
    assert np.array_equal(bits((y1 * 2).astype(np.float16)), bits(y2))


def test_graph_replay_and_dependent_launch(gpu):
    # a recorded step replays bit-identically, with and without programmatic dependent launch
    from mlxl3_b200.runtime import DeviceBuffer, Graph, Stream
    rng = np.random.default_rng(31)
    layers, wants = [], []
    x = rng.standard_normal((2, 1024)).astype(np.float16)
    for i in range(6):
        trellis, suh, svh = random_layer(rng, 1024, 1024, 4)
        svh = (svh.astype(np.float32) / 32).astype(np.float16)       # keep the chain's magnitude at O(1)
        layers.append(gpu.Exl3Linear(trellis, suh, svh, None, 4, 0))
    stream = Stream()
    d_x = DeviceBuffer.from_numpy(x)
    d_y = [DeviceBuffer(2 * 1024 * 2) for _ in layers]
    ws = gpu.new_workspace(max(l.workspace_bytes(2) for l in layers))

    def step():
        src = d_x
        for layer, dst in zip(layers, d_y):           # a chain: each layer consumes the previous output
            layer.forward_device(src.ptr, gpu.F16, 2, dst.ptr, ws, stream)
            src = dst

    step()
    stream.sync()
    eager = [d.download((2, 1024), np.float16, stream) for d in d_y]
    assert np.isfinite(eager[-1].astype(np.float32)).all()
    for pdl in (0, 1, 2):
        gpu.set_option("pdl", pdl)
        try:
            step()                                         # warm
            with Graph.record(stream) as graph:
                step()
            for d in d_y:
                d.fill(0, stream)
            graph.launch(stream)
            graph.launch(stream)
            stream.sync()
            for want, d in zip(eager, d_y):
                assert np.array_equal(bits(d.download((2, 1024), np.float16, stream)), bits(want))
            assert gpu.workspace_status(ws) == 0
        finally:
            gpu.set_option("pdl", 0)
