"""A decode step as one persistent launch (Exl3Stack) against the same layers launched one by one.

The step kernel computes every layer with the arithmetic and the summation order of the per-layer kernel, so for the
same work partition the outputs are the same bits; the partition differs only in how many warps share a layer (the
per-layer launch sizes its grid per layer), so the stated bar against the per-layer path is the accumulation-order
bar of the layer tests (RMS difference below 1e-3 of the output RMS), and the bar against the CPU oracle is the layer
bar (max |got - oracle| <= 1e-2 * max|oracle| per row).  Replays of one stack must be bit-identical.
"""
import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu, random_layer  # noqa: F401

pytestmark = pytest.mark.gpu


def _rms(a):
    return float(np.sqrt((np.asarray(a, np.float64) ** 2).mean()))


def _close(got, want, rms=1e-3):
    g, w = got.astype(np.float32), want.astype(np.float32)
    assert g.shape == w.shape and np.isfinite(g).all()
    scale = np.abs(w).max(axis=1, keepdims=True)
    assert (np.abs(g - w) <= 1e-2 * scale).all(), float((np.abs(g - w) / scale).max())
    assert _rms(g - w) <= rms * _rms(w), _rms(g - w) / _rms(w)


@pytest.mark.parametrize("k,cb,rows,exact", [(4, 0, 1, False), (4, 0, 2, True), (3, 1, 1, False), (2, 2, 2, False), (6, 0, 2, True),
                                             (8, 1, 1, False), (5, 2, 2, False), (1, 0, 1, True), (7, 1, 1, False)])
def test_chain_of_layers_matches_per_layer_calls_and_oracle(gpu, k, cb, rows, exact):
    """A chain x -> L0 -> L1 -> ... where every layer consumes the previous layer's output, widths that change
    from layer to layer (more and fewer column blocks than CTAs per layer), and one grouped layer in the middle."""
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    rng = np.random.default_rng(100 * k + 10 * cb + rows)
    widths = [512, 1024, 384, 2048, 128, 512]
    stream = Stream()
    layers, host = [], []
    for n_in, n_out in zip(widths[:-1], widths[1:]):
        trellis, suh, svh = random_layer(rng, n_in, n_out, k)
        svh = (svh.astype(np.float32) / np.sqrt(n_in)).astype(np.float16)      # keep the chain's magnitude at O(1)
        bias = (rng.standard_normal(n_out) * 0.05).astype(np.float16) if n_out == 384 else None
        host.append((trellis, suh, svh, bias))
        layers.append(gpu.Exl3Linear(trellis, suh, svh, bias, k, cb, exact_weights=exact))
    # a grouped layer (two members that read the last output) at the end of the chain
    members_host = []
    for n_out in (256, 128):
        trellis, suh, svh = random_layer(rng, widths[-1], n_out, k)
        svh = (svh.astype(np.float32) / np.sqrt(widths[-1])).astype(np.float16)
        members_host.append((trellis, suh, svh))
    members = [gpu.Exl3Linear(t, s, v, None, k, cb, exact_weights=exact) for t, s, v in members_host]
    group = gpu.Exl3Group(members)
    x = rng.standard_normal((rows, widths[0])).astype(np.float16)
    d_x = DeviceBuffer.from_numpy(x)
    d_y = [DeviceBuffer(rows * w * 2) for w in widths[1:]]
    d_g = [DeviceBuffer(rows * 256 * 2), DeviceBuffer(rows * 128 * 2)]
    ws = gpu.new_workspace(max([l.workspace_bytes(rows) for l in layers] + [group.workspace_bytes(rows)]))

    # per-layer calls
    src = d_x
    for layer, dst in zip(layers, d_y):
        layer.forward_device(src.ptr, gpu.F16, rows, dst.ptr, ws, stream)
        src = dst
    group.forward_device(src.ptr, gpu.F16, rows, [d.ptr for d in d_g], ws, stream)
    stream.sync()
    want = [d.download((rows, w), np.float16, stream) for d, w in zip(d_y, widths[1:])]
    want_g = [d.download((rows, w), np.float16, stream) for d, w in zip(d_g, (256, 128))]
    assert gpu.workspace_status(ws) == 0

    # the same step as one launch, into fresh buffers
    s_y = [DeviceBuffer(rows * w * 2) for w in widths[1:]]
    s_g = [DeviceBuffer(rows * 256 * 2), DeviceBuffer(rows * 128 * 2)]
    ops, src = [], d_x
    for layer, dst in zip(layers, s_y):
        ops.append((layer, src.ptr, dst.ptr))
        src = dst
    ops.append((group, src.ptr, [d.ptr for d in s_g]))
    stack = gpu.Exl3Stack(ops, gpu.F16, rows)
    replays = []
    for _ in range(3):
        for d in s_y + s_g:
            d.fill(0xFF, stream)
        stack.forward(stream)
        stream.sync()
        assert stack.status() == 0
        replays.append([d.download((rows, w), np.float16, stream) for d, w in zip(s_y + s_g, widths[1:] + [256, 128])])
    for other in replays[1:]:
        for a, b in zip(replays[0], other):
            assert np.array_equal(bits(a), bits(b))
    got = replays[0]
    # against the per-layer path: layer by layer the inputs are (nearly) the same, so compare the whole chain loosely
    # and the first layer tightly
    _close(got[0], want[0])
    for g_, w_ in zip(got, want + want_g):
        _close(g_, w_, rms=2e-2)
    # against the oracle, layer by layer ON THE STEP'S OWN INPUTS (each layer's input is the step's previous output)
    prev = x
    for (trellis, suh, svh, bias), out in zip(host, got[:len(host)]):
        _close(out, oracle.linear_forward(trellis, k, cb, suh, svh, bias, prev), rms=4e-3)
        prev = out
    for (trellis, suh, svh), out in zip(members_host, got[len(host):]):
        _close(out, oracle.linear_forward(trellis, k, cb, suh, svh, None, prev), rms=4e-3)
    stack.close()


def test_step_of_full_size_layers(gpu):
    """One decoder layer's projections at their real sizes (4 bits): [q|k|v] group, o, [gate|up] group, down, each on
    its own input buffer, all in one launch; sampled against the oracle."""
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    rng = np.random.default_rng(8)
    hidden, ffn, kv, k, cb = 4096, 14336, 1024, 4, 0
    stream = Stream()

    def make(n_in, n_out):
        t, s, v = random_layer(rng, n_in, n_out, k)
        return (t, s, v), gpu.Exl3Linear(t, s, v, None, k, cb)
    qkv = [make(hidden, n) for n in (hidden, kv, kv)]
    o = make(hidden, hidden)
    gu = [make(hidden, ffn) for _ in range(2)]
    down = make(ffn, hidden)
    g_qkv, g_gu = gpu.Exl3Group([l for _, l in qkv]), gpu.Exl3Group([l for _, l in gu])
    x_h = rng.standard_normal((1, hidden)).astype(np.float16)
    x_f = rng.standard_normal((1, ffn)).astype(np.float16)
    d_h, d_f = DeviceBuffer.from_numpy(x_h), DeviceBuffer.from_numpy(x_f)
    out = {name: DeviceBuffer(n * 2) for name, n in (("q", hidden), ("k", kv), ("v", kv), ("o", hidden), ("gate", ffn), ("up", ffn), ("down", hidden))}
    stack = gpu.Exl3Stack([(g_qkv, d_h.ptr, [out["q"].ptr, out["k"].ptr, out["v"].ptr]), (o[1], d_h.ptr, out["o"].ptr),
                           (g_gu, d_h.ptr, [out["gate"].ptr, out["up"].ptr]), (down[1], d_f.ptr, out["down"].ptr)], gpu.F16, 1)
    grid, smem = stack.geometry()
    assert grid >= 148 and smem <= 224 * 1024
    stack.forward(stream)
    stack.forward(stream)
    stream.sync()
    assert stack.status() == 0
    cases = [("q", qkv[0][0], x_h), ("k", qkv[1][0], x_h), ("v", qkv[2][0], x_h), ("o", o[0], x_h), ("gate", gu[0][0], x_h),
             ("up", gu[1][0], x_h), ("down", down[0], x_f)]
    for name, (t, s, v), x in cases:
        got = out[name].download((1, t.shape[1] * 16), np.float16, stream)
        _close(got, oracle.linear_forward(t, k, cb, s, v, None, x), rms=2e-3)
    stack.close()


def test_step_validation(gpu):
    from mlxl3_b200.runtime import DeviceBuffer
    rng = np.random.default_rng(3)
    a = gpu.Exl3Linear(*random_layer(rng, 256, 256, 4), None, 4, 0)
    b = gpu.Exl3Linear(*random_layer(rng, 256, 256, 3), None, 3, 0)
    d = DeviceBuffer(4 * 256 * 2)
    with pytest.raises(gpu.B200Exl3Error, match="share bit width"):
        gpu.Exl3Stack([(a, d.ptr, d.ptr), (b, d.ptr, d.ptr)], gpu.F16, 1)
    with pytest.raises(gpu.B200Exl3Error, match="1 to 2 activation rows"):
        gpu.Exl3Stack([(a, d.ptr, d.ptr)], gpu.F16, 3)
    with pytest.raises(gpu.B200Exl3Error, match="NULL or not 16-byte aligned"):
        gpu.Exl3Stack([(a, d.ptr + 2, d.ptr)], gpu.F16, 1)
    with pytest.raises(gpu.B200Exl3Error, match="between 1 and 256"):
        gpu.Exl3Stack([], gpu.F16, 1)
