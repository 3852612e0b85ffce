"""GPU parity at the shapes the benchmark configurations name, each against the CPU oracle on the same seeded
inputs (the oracle on a sample of rows where a full CPU product would take minutes):

* grouped experts, 128 experts / top-8 / 2048 <-> 768 / 3 bits: one token (one row per slot) and 256 tokens
  (64-row tensor-core segments), plus an expert id of 0xFFFFFFFF, which must be clamped, not dereferenced;
* the dense MLP block at 512 rows and 3 bits: the gate|up pair 4096 -> (14336, 14336) as one group and the
  down projection 14336 -> 4096 (tensor-core product with a split input range, then the output rotation);
* the 16-row verify shapes 5120 -> 25600, 25600 -> 5120, 5120 -> 8192, 8192 -> 5120 at 2, 3, 4 and 6 bits and
  their shards for a tensor-parallel group of eight through the exchange entry point with a world of one.

Bars: those of the small-shape tests -- max |got - oracle| <= 1e-2 * max|oracle| per row, and an RMS difference
below 2e-3 of the output RMS (default split-weight mode for the dense layers, exact weights for the experts).
"""
import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu, random_layer  # noqa: F401
from tests.test_gpu_moe import check as check_moe, make_bank, routes

pytestmark = pytest.mark.gpu


def _check(got, want, rms=2e-3):
    g, w = got.astype(np.float32), want.astype(np.float32)
    assert g.shape == w.shape and np.isfinite(g).all()
    scale = np.abs(w).max(axis=1, keepdims=True)
    assert (np.abs(g - w) <= 1e-2 * scale).all(), float((np.abs(g - w) / scale).max())
    assert np.sqrt(((g - w) ** 2).mean()) <= rms * np.sqrt((w ** 2).mean())


@pytest.fixture(scope="module")
def expert_bank():
    rng = np.random.default_rng(4004)
    return make_bank(rng, 128, 2048, 768, 3)


def test_expert_block_one_token(gpu, expert_bank):
    rng = np.random.default_rng(4005)
    moe = gpu.Exl3SwitchGlu(*expert_bank, 8, 3, 0, exact_weights=True)
    x = rng.standard_normal((1, 2048)).astype(np.float16)
    selected, scores = routes(rng, 1, 128, 8)
    got = moe.forward(x, selected, scores)
    check_moe(got, oracle.switch_glu_forward(*expert_bank, 8, 3, 0, x, selected, scores))
    assert gpu.workspace_status(moe._workspace) == 0
    assert np.array_equal(bits(got), bits(moe.forward(x, selected, scores)))
    # an id beyond the bank (here the largest 32-bit value) is clamped to the last expert, as an id of `experts` is
    wild = selected.copy()
    wild[0, 3] = 0xFFFFFFFF
    tame = selected.copy()
    tame[0, 3] = 127
    assert np.array_equal(bits(moe.forward(x, wild, scores)), bits(moe.forward(x, tame, scores)))
    assert gpu.workspace_status(moe._workspace) == 0
    moe.close()


def test_expert_block_256_tokens(gpu, expert_bank):
    rng = np.random.default_rng(4006)
    moe = gpu.Exl3SwitchGlu(*expert_bank, 8, 3, 0, exact_weights=True)
    x = rng.standard_normal((256, 2048)).astype(np.float16)
    selected, scores = routes(rng, 256, 128, 8)
    selected[17, 5] = 0xFFFFFFFF                               # clamped to expert 127 by the route plan
    got = moe.forward(x, selected, scores)
    assert gpu.workspace_status(moe._workspace) == 0
    assert np.isfinite(got.astype(np.float32)).all()
    pick = np.array([0, 17, 63, 64, 128, 200, 254, 255])
    sel = selected[pick].copy()
    sel[sel == 0xFFFFFFFF] = 127
    check_moe(got[pick], oracle.switch_glu_forward(*expert_bank, 8, 3, 0, x[pick], sel, scores[pick]))
    assert np.array_equal(bits(got), bits(moe.forward(x, selected, scores)))
    # 64 tokens of the same batch take the 8-row segments of the fused kernel: same rows, other summation order
    small = moe.forward(x[:64], selected[:64], scores[:64])
    check_moe(small[[0, 17, 63]], got[[0, 17, 63]])
    moe.close()


def test_mlp_block_512_rows(gpu):
    rng = np.random.default_rng(2001)
    rows, k, cb, hidden, ffn = 512, 3, 0, 4096, 14336
    x = rng.standard_normal((rows, hidden)).astype(np.float16)
    pick = np.array([0, 255, 256, 511])
    gate_w, up_w = random_layer(rng, hidden, ffn, k), random_layer(rng, hidden, ffn, k)
    gate, up = (gpu.Exl3Linear(*w, None, k, cb) for w in (gate_w, up_w))
    group = gpu.Exl3Group([gate, up])
    outs = group.forward(x)
    for got, w, single in zip(outs, (gate_w, up_w), (gate, up)):
        _check(got[pick], oracle.linear_forward(w[0], k, cb, w[1], w[2], None, x[pick]))
    # the pair as a group and each member alone agree to summation order
    _check(outs[0][pick], gate.forward(x)[pick], rms=1e-3)
    group.close(), gate.close(), up.close()
    # down projection: the activation is SwiGLU of the two products, scaled back to O(1)
    g32, u32 = outs[0].astype(np.float32) / 64, outs[1].astype(np.float32) / 64
    act = (g32 / (1 + np.exp(-g32)) * u32).astype(np.float16)
    down_w = random_layer(rng, ffn, hidden, k)
    down = gpu.Exl3Linear(*down_w, None, k, cb)
    y = down.forward(act)
    assert gpu.workspace_status(down._workspace) == 0
    _check(y[pick], oracle.linear_forward(down_w[0], k, cb, down_w[1], down_w[2], None, act[pick]))
    assert np.array_equal(bits(y), bits(down.forward(act)))
    down.close()


VERIFY_SHAPES = [(5120, 25600, 2), (25600, 5120, 3), (5120, 8192, 4), (8192, 5120, 6)]


@pytest.mark.parametrize("n_in,n_out,k", VERIFY_SHAPES)
def test_verify_width_16_full_layers(gpu, n_in, n_out, k):
    rng = np.random.default_rng(5000 + k)
    trellis, suh, svh = random_layer(rng, n_in, n_out, k)
    x = rng.standard_normal((16, n_in)).astype(np.float16)
    layer = gpu.Exl3Linear(trellis, suh, svh, None, k, 0)
    got = layer.forward(x)
    assert gpu.workspace_status(layer._workspace) == 0
    _check(got, oracle.linear_forward(trellis, k, 0, suh, svh, None, x))
    layer.close()


@pytest.mark.parametrize("n_in,n_out,k,kind", [(5120, 25600, 3, "col"), (25600, 5120, 2, "row"), (5120, 8192, 6, "col"),
                                               (8192, 5120, 4, "row")])
def test_verify_width_16_shards_of_eight(gpu, n_in, n_out, k, kind):
    """One rank's shard of a tensor-parallel group of eight (25600 / 8 = 3200 = 25 blocks of 128)."""
    from mlxl3_b200 import tp
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    rng = np.random.default_rng(5100 + k)
    s_in, s_out = tp.shard_dims(kind, n_in, n_out, 8)
    trellis, suh, svh = random_layer(rng, s_in, s_out, k)
    x = rng.standard_normal((16, s_in)).astype(np.float16)
    want = oracle.linear_forward(trellis, k, 0, suh, svh, None, x)
    layer = gpu.Exl3Linear(trellis, suh, svh, None, k, 0)
    if kind == "col":
        _check(layer.forward(x), want)
    else:
        # row shard: the fused kernel with the exchange of the block sums inside it; with a world of one the rank
        # exchanges with itself, so the result is the plain layer output
        stream = Stream()
        ctx = tp.TpContext(0, 1, 16 * s_out // 128, lambda raw: [raw])
        d_x, d_y = DeviceBuffer.from_numpy(x), DeviceBuffer(16 * s_out * 2)
        ws = gpu.new_workspace(layer.workspace_bytes(16))
        for _ in range(2):
            d_y.fill(0, stream)
            ctx.forward(layer, d_x.ptr, gpu.F16, 16, d_y.ptr, ws, stream)
            _check(d_y.download((16, s_out), np.float16, stream), want)
        assert ctx.status() == 0 and gpu.workspace_status(ws) == 0
        ctx.close()
    layer.close()
