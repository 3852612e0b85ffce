"""GPU parity of the grouped-expert SwiGLU block (Exl3SwitchGlu.forward) through the C ABI.

The oracle runs the reference's chain slot by slot.  What may differ on the GPU: the fp32 summation
order of the three products, and the last bits of exp() inside SiLU (the reference's Metal exp is a
fast-math intrinsic, so that step is not pinned).  Stated bar: max |got - oracle| <= 1e-2 * max|oracle|
per row and an RMS difference below 2e-3 of the output RMS.
"""
import numpy as np
import pytest

import oracle
from tests.gpu_util import gpu  # noqa: F401

pytestmark = pytest.mark.gpu


def make_bank(rng, experts, n_in, hidden, k):
    gu_t = rng.integers(0, 65536, (n_in // 16, experts * hidden // 8, 16 * k), dtype=np.uint16)
    down_t = rng.integers(0, 65536, (hidden // 16, experts * n_in // 16, 16 * k), dtype=np.uint16)
    sign = lambda *shape: np.where(rng.random(shape) > 0.5, -1, 1).astype(np.float16)  # noqa: E731
    # the inner matrices have unit-variance entries: scale the outputs down so that activations stay O(1)
    gu_svh = (sign(experts, 2, hidden).astype(np.float32) * rng.uniform(0.5, 1.5, (experts, 2, hidden)) / np.sqrt(n_in)).astype(np.float16)
    down_svh = (sign(experts, n_in).astype(np.float32) * rng.uniform(0.5, 1.5, (experts, n_in)) / np.sqrt(hidden)).astype(np.float16)
    return gu_t, sign(experts, 2, n_in), gu_svh, down_t, sign(experts, hidden), down_svh


def routes(rng, rows, experts, top_k):
    selected = np.stack([rng.permutation(experts)[:top_k] for _ in range(rows)]).astype(np.uint32)
    scores = rng.random((rows, top_k)).astype(np.float32)
    scores /= scores.sum(axis=1, keepdims=True)
    return selected, scores.astype(np.float16)


def check(got, want, rms=2e-3):
    g, w = got.astype(np.float32), want.astype(np.float32)
    assert g.shape == w.shape and np.isfinite(g).all()
    scale = np.abs(w).max(axis=1, keepdims=True)
    assert (np.abs(g - w) <= 1e-2 * scale).all(), float((np.abs(g - w) / scale).max())
    assert np.sqrt(((g - w) ** 2).mean()) <= rms * np.sqrt((w ** 2).mean())


@pytest.mark.parametrize("k,cb,experts,top_k,n_in,hidden,rows", [
    (3, 1, 8, 2, 256, 128, 1), (4, 0, 16, 4, 256, 384, 3), (2, 2, 4, 4, 384, 256, 2), (5, 0, 8, 3, 128, 256, 5),
    (8, 1, 4, 1, 256, 128, 2), (1, 0, 6, 2, 128, 128, 4), (6, 2, 5, 5, 256, 256, 1)])
def test_switch_glu_matches_oracle(gpu, k, cb, experts, top_k, n_in, hidden, rows):
    rng = np.random.default_rng(9000 + 100 * k + 10 * cb + rows)
    bank = make_bank(rng, experts, n_in, hidden, k)
    moe = gpu.Exl3SwitchGlu(*bank, top_k, k, cb, exact_weights=True)
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    selected, scores = routes(rng, rows, experts, top_k)
    want = oracle.switch_glu_forward(*bank, top_k, k, cb, x, selected, scores)
    got = moe.forward(x, selected, scores)
    assert got.dtype == np.float16
    check(got, want)
    assert gpu.workspace_status(moe._workspace) == 0
    # same call again: bit-identical; fp32 routing weights give an fp32 result close to the fp16 one
    assert np.array_equal(got.view(np.uint16), moe.forward(x, selected, scores).view(np.uint16))
    got32 = moe.forward(x, selected, scores.astype(np.float32))
    assert got32.dtype == np.float32
    check(got32, want, rms=3e-3)
    # default (split-weight) mode stays inside the same bars
    fast = gpu.Exl3SwitchGlu(*bank, top_k, k, cb)
    check(fast.forward(x, selected, scores), want, rms=4e-3)
    fast.close()
    moe.close()


def test_switch_glu_many_rows_and_repeated_experts(gpu):
    """600 slots over 12 experts (50 per expert): the expert-sorted form with segments of 64 rows through the
    tensor-core product, every expert chosen many times, and experts that nobody chose."""
    rng = np.random.default_rng(77)
    experts, top_k, n_in, hidden, k, cb, rows = 12, 4, 256, 256, 3, 1, 150
    bank = make_bank(rng, experts, n_in, hidden, k)
    moe = gpu.Exl3SwitchGlu(*bank, top_k, k, cb, exact_weights=True)
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    selected, scores = routes(rng, rows, experts - 2, top_k)          # the last two experts stay idle
    got = moe.forward(x, selected, scores)
    assert gpu.workspace_status(moe._workspace) == 0
    pick = np.array([0, 1, 63, 64, 65, 127, 128, 149])
    want = oracle.switch_glu_forward(*bank, top_k, k, cb, x[pick], selected[pick], scores[pick])
    check(got[pick], want)
    # same call again: bit-identical (a slot's place inside its segment may change, its arithmetic does not)
    assert np.array_equal(got.view(np.uint16), moe.forward(x, selected, scores).view(np.uint16))
    # one row per slot (sorting switched off) agrees to accumulation order
    gpu.set_option("moe_sorted", 0)
    try:
        plain = moe.forward(x, selected, scores)
    finally:
        gpu.set_option("moe_sorted", 1)
    check(got, plain, rms=2e-3)
    # a row computed alone (few slots: one row per slot) matches its result inside the batch
    alone = moe.forward(x[64:65], selected[64:65], scores[64:65])
    check(alone, got[64:65], rms=2e-3)
    moe.close()


@pytest.mark.parametrize("rows,top_k,experts", [(9, 4, 4), (40, 1, 3), (80, 2, 32)])
def test_switch_glu_sorted_edge_shapes(gpu, rows, top_k, experts):
    """Segments that are exactly full, a single expert taking every slot, many experts with few rows each."""
    rng = np.random.default_rng(1000 + rows)
    n_in, hidden, k, cb = 128, 128, 4, 0
    bank = make_bank(rng, experts, n_in, hidden, k)
    moe = gpu.Exl3SwitchGlu(*bank, top_k, k, cb, exact_weights=True)
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    selected, scores = routes(rng, rows, experts, top_k)
    if experts == 3:
        selected[:] = 1                                               # everybody picks the same expert
    got = moe.forward(x, selected, scores)
    check(got, oracle.switch_glu_forward(*bank, top_k, k, cb, x, selected, scores))
    assert gpu.workspace_status(moe._workspace) == 0
    moe.close()


def test_switch_glu_validation(gpu):
    rng = np.random.default_rng(5)
    bank = make_bank(rng, 4, 128, 128, 2)
    with pytest.raises(gpu.B200Exl3Error, match="invalid or overflowing SwitchGLU dimensions"):
        gpu.Exl3SwitchGlu(*bank, 5, 2, 0)                       # top_k > experts
    with pytest.raises(gpu.B200Exl3Error, match="SwitchGLU trellis/scales disagree"):
        gpu.Exl3SwitchGlu(bank[0], bank[1], bank[2], bank[3], bank[4][:, :64], bank[5], 2, 2, 0)
    moe = gpu.Exl3SwitchGlu(*bank, 2, 2, 0)
    with pytest.raises(gpu.B200Exl3Error, match="invalid SwitchGLU input/routes"):
        moe.forward(np.zeros((2, 128), np.float16), np.zeros((2, 3), np.uint32), np.zeros((2, 3), np.float16))
    with pytest.raises(gpu.B200Exl3Error, match="SwitchGLU input must have rank 2"):
        moe.forward(np.zeros(128, np.float16), np.zeros((1, 2), np.uint32), np.zeros((1, 2), np.float16))
    moe.close()


@pytest.mark.parametrize("pdl", [1, 2])
def test_routes_written_by_the_previous_kernel_under_dependent_launch(gpu, pdl):
    """Router and expert block alternate on one stream with programmatic dependent launch switched on and routes
    that change every iteration: the expert kernels must read the routes the router has just written, never the
    previous iteration's (they wait for the previous kernel's memory before touching them)."""
    from mlxl3_b200 import router
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    from oracle import router as oracle_router
    rng = np.random.default_rng(60 + pdl)
    experts, top_k, n_in, hidden, k, cb = 16, 4, 256, 256, 4, 0
    bank = make_bank(rng, experts, n_in, hidden, k)
    moe = gpu.Exl3SwitchGlu(*bank, top_k, k, cb, exact_weights=True)
    stream = Stream()
    ws = gpu.new_workspace(moe.workspace_bytes(1))
    d_sel, d_scores, d_y = DeviceBuffer(top_k * 4), DeviceBuffer(top_k * 2), DeviceBuffer(n_in * 2)
    iters = 6
    xs = rng.standard_normal((iters, 1, n_in)).astype(np.float16)
    logits = (rng.standard_normal((iters, 1, experts)) * 2).astype(np.float16)
    d_xs = [DeviceBuffer.from_numpy(x) for x in xs]
    d_logits = [DeviceBuffer.from_numpy(v) for v in logits]
    d_ys = [DeviceBuffer(n_in * 2) for _ in range(iters)]
    gpu.set_option("pdl", pdl)
    try:
        for i in range(iters):                         # back to back, no host synchronisation in between
            router.topk_device(d_logits[i].ptr, gpu.F16, 1, experts, top_k, True, d_sel.ptr, d_scores.ptr, stream)
            moe.forward_device(d_xs[i].ptr, gpu.F16, 1, d_sel.ptr, d_scores.ptr, gpu.F16, d_ys[i].ptr, ws, stream)
        stream.sync()
    finally:
        gpu.set_option("pdl", 0)
    assert gpu.workspace_status(ws) == 0
    for i in range(iters):
        sel, scores = oracle_router.topk(logits[i], top_k, True)
        want = oracle.switch_glu_forward(*bank, top_k, k, cb, xs[i], sel, scores)
        check(d_ys[i].download((1, n_in), np.float16, stream), want)
    moe.close()


@pytest.mark.parametrize("k,cb,experts,top_k,n_in,hidden,rows", [(3, 0, 16, 8, 256, 384, 1), (4, 1, 8, 2, 384, 128, 3), (5, 2, 6, 3, 128, 256, 7)])
def test_small_batch_glue_fused_into_the_down_product(gpu, k, cb, experts, top_k, n_in, hidden, rows):
    """Two launches (the down product takes the SwiGLU glue as its prologue and the weighted reduction as its epilogue)
    against four: the same arithmetic in the same order, so the same bits, for fp16 and fp32 routing weights."""
    rng = np.random.default_rng(4400 + 10 * k + rows)
    bank = make_bank(rng, experts, n_in, hidden, k)
    moe = gpu.Exl3SwitchGlu(*bank, top_k, k, cb)
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    selected, scores = routes(rng, rows, experts, top_k)
    want = oracle.switch_glu_forward(*bank, top_k, k, cb, x, selected, scores)
    for s in (scores, scores.astype(np.float32)):
        four = moe.forward(x, selected, s)
        gpu.set_option("moe_fused", 1)
        try:
            two = moe.forward(x, selected, s)
            again = moe.forward(x, selected, s)                # the counters were left at zero
        finally:
            gpu.set_option("moe_fused", 0)
        assert two.dtype == four.dtype and np.array_equal(two.view(np.uint8), four.view(np.uint8))
        assert np.array_equal(two.view(np.uint8), again.view(np.uint8))
        check(two, want, rms=4e-3)
    assert gpu.workspace_status(moe._workspace) == 0
