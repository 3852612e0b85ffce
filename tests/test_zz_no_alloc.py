"""The allocation-free forward entry point (scratch in a fixed array inside the library) must give what
the workspace-based entry point gives.  Collected last on purpose: a failure here cannot hide another."""
import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu, random_layer  # noqa: F401
from tests.test_gpu_linear import _check_out

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows", [1, 5, 24])   # 24 rows: the tensor-core product also runs on the static scratch
def test_static_scratch_forward_matches_workspace_forward(gpu, rows):
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    rng = np.random.default_rng(4100 + rows)
    trellis, suh, svh = random_layer(rng, 1024, 512, 4)
    bias = (rng.standard_normal(512) * 0.1).astype(np.float16)
    layer = gpu.Exl3Linear(trellis, suh, svh, bias, 4, 0)
    stream = Stream()
    ws = gpu.new_workspace(layer.workspace_bytes(rows))
    d_y_ref, d_y = DeviceBuffer(rows * 512 * 2), DeviceBuffer(rows * 512 * 2)
    for call in range(2):                                   # two calls in a row share the one scratch array
        x = rng.standard_normal((rows, 1024)).astype(np.float16)
        d_x = DeviceBuffer.from_numpy(x, stream)
        layer.forward_device(d_x.ptr, gpu.F16, rows, d_y_ref.ptr, ws, stream)
        d_y.fill(0xFF, stream)
        layer.forward_static_device(d_x.ptr, gpu.F16, rows, d_y.ptr, stream)
        want = d_y_ref.download((rows, 512), np.float16, stream)
        got = d_y.download((rows, 512), np.float16, stream)
        assert np.isfinite(got.astype(np.float32)).all()
        _check_out(got, want)                               # the tolerance of the layer tests ...
        assert np.array_equal(bits(got), bits(want))        # ... and in fact the same bits: same kernel, same plan
        _check_out(got, oracle.linear_forward(trellis, 4, 0, suh, svh, bias, x))
        assert gpu.static_status() == 0                     # no bounded wait gave up on the shared array


def test_static_scratch_rejects_oversized_calls(gpu):
    from mlxl3_b200.runtime import DeviceBuffer
    rng = np.random.default_rng(7)
    trellis, suh, svh = random_layer(rng, 2048, 28672, 2)
    layer = gpu.Exl3Linear(trellis, suh, svh, None, 2, 0)
    rows = 256
    assert layer.workspace_bytes(rows) > 4 << 20
    d_x, d_y = DeviceBuffer(rows * 2048 * 2), DeviceBuffer(rows * 28672 * 2)
    with pytest.raises(gpu.B200Exl3Error, match="allocation-free entry point owns"):
        layer.forward_static_device(d_x.ptr, gpu.F16, rows, d_y.ptr)
    # a small call on the same layer still works afterwards
    x = rng.standard_normal((1, 2048)).astype(np.float16)
    d_x1, d_y1 = DeviceBuffer.from_numpy(x), DeviceBuffer(28672 * 2)
    layer.forward_static_device(d_x1.ptr, gpu.F16, 1, d_y1.ptr)
    _check_out(d_y1.download((1, 28672), np.float16), oracle.linear_forward(trellis, 2, 0, suh, svh, None, x))
