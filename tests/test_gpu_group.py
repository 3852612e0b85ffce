"""GPU parity of Exl3Group (projections that share their input, one launch) through the C ABI."""
import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu, random_layer  # noqa: F401
from tests.test_gpu_linear import _check_out

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k,cb", [(4, 0), (3, 1), (5, 2), (7, 0)])
def test_group_matches_oracle(gpu, k, cb):
    rng = np.random.default_rng(700 + k)
    n_in, widths = 1024, (512, 128, 256)
    members, params = [], []
    for i, w in enumerate(widths):
        trellis, suh, svh = random_layer(rng, n_in, w, k, signs=(i != 1))
        bias = (rng.standard_normal(w) * 0.2).astype(np.float16) if i == 2 else None
        params.append((trellis, suh, svh, bias))
        members.append(gpu.Exl3Linear(trellis, suh, svh, bias, k, cb, exact_weights=True))
    assert gpu.Exl3Group.compatible(members)
    group = gpu.Exl3Group(members)
    for m in members:                               # the group owns copies: members may go away
        m.close()
    for rows in (1, 2, 5, 20):
        x = rng.standard_normal((rows, n_in)).astype(np.float16)
        outs = group.forward(x)
        assert len(outs) == 3
        for (trellis, suh, svh, bias), w, y in zip(params, widths, outs):
            assert y.shape == (rows, w) and y.dtype == np.float16
            _check_out(y, oracle.linear_forward(trellis, k, cb, suh, svh, bias, x))
    x32 = rng.standard_normal((3, n_in)).astype(np.float32)
    outs32 = group.forward(x32)
    for (trellis, suh, svh, bias), y in zip(params, outs32):
        assert y.dtype == np.float32
        _check_out(y, oracle.linear_forward(trellis, k, cb, suh, svh, bias, x32))


def test_group_rules(gpu):
    rng = np.random.default_rng(9)
    a = gpu.Exl3Linear(*random_layer(rng, 256, 128, 4), None, 4, 0)
    b = gpu.Exl3Linear(*random_layer(rng, 256, 256, 4), None, 4, 0)
    c = gpu.Exl3Linear(*random_layer(rng, 128, 128, 4), None, 4, 0)       # other input width
    d = gpu.Exl3Linear(*random_layer(rng, 256, 128, 3), None, 3, 0)       # other K
    e = gpu.Exl3Linear(*random_layer(rng, 256, 128, 4), None, 4, 1)       # other codebook
    assert gpu.Exl3Group.compatible([a, b])
    for bad in ([a], [a, c], [a, d], [a, e], []):
        assert not gpu.Exl3Group.compatible(bad)
        with pytest.raises(gpu.B200Exl3Error, match="incompatible grouped projections"):
            gpu.Exl3Group(bad)
    group = gpu.Exl3Group([a, b])
    with pytest.raises(gpu.B200Exl3Error, match="invalid grouped EXL3 input"):
        group.forward(np.zeros((1, 128), np.float16))
    # the fused call equals the separate calls within the accumulation-order noise
    x = rng.standard_normal((2, 256)).astype(np.float16)
    ya, yb = group.forward(x)
    _check_out(ya, a.forward(x), rel=2e-3)
    _check_out(yb, b.forward(x), rel=2e-3)
