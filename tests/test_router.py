"""Stable top-k router: the oracle's properties on CPU, GPU parity through the C ABI (bit-exact: index work and
a fixed-order sum)."""
import numpy as np
import pytest

from oracle import router as oracle_router
from tests.gpu_util import gpu  # noqa: F401


def test_oracle_order_ties_and_specials():
    values = np.array([[0.5, 2.0, 2.0, -1.0, 0.0, -0.0, np.nan, 1.0]], np.float32)
    indices, scores = oracle_router.topk(values, 4, False)
    # ascending, best last: NaN ranks above every number; of the two 2.0 the higher index ranks higher
    assert indices.tolist() == [[7, 1, 2, 6]]
    assert np.array_equal(scores[0, :3], np.array([1.0, 2.0, 2.0], np.float32)) and np.isnan(scores[0, 3])
    # +0 and -0 compare equal: the higher index wins the tie
    indices, _ = oracle_router.topk(np.array([[0.0, -0.0, -1.0]], np.float16), 1, False)
    assert indices.tolist() == [[1]]
    # normalisation adds in slot order in the values' own type
    v = np.array([[0.1, 0.7, 0.2, 0.05]], np.float16)
    indices, scores = oracle_router.topk(v, 3, True)
    assert indices.tolist() == [[0, 2, 1]]
    total = np.float16(np.float16(np.float16(0.1) + np.float16(0)) + np.float16(0))
    total = np.float16(np.float16(0.2) + np.float16(np.float16(0.1) + np.float16(0)))
    total = np.float16(np.float16(0.7) + total)
    assert np.array_equal(scores[0], (np.array([0.1, 0.2, 0.7], np.float16) / total).astype(np.float16))


def _reference_case():
    """The inputs and expected outputs of the reference's own router test
    (native/src/router.rs:427-466: float_router_preserves_precision_ties_and_boundaries)."""
    values = np.array([0.2 + ((i * 7) % 17) * 0.000001 for i in range(34)], np.float32).reshape(2, 17)
    cases = []
    for k in (1, 10, 17):
        expected = np.stack([np.array(sorted(range(17), key=lambda a: (values[row, a], a))[17 - k:], np.uint32) for row in range(2)])
        cases.append((k, expected))
    return values, cases


def test_oracle_reproduces_the_reference_router_test():
    values, cases = _reference_case()
    for k, expected in cases:
        ids, scores = oracle_router.topk(values, k, True)
        assert scores.dtype == np.float32 and np.array_equal(ids, expected)
        for row in range(2):
            total = values[row, expected[row]].sum(dtype=np.float32)
            assert np.abs(scores[row] - values[row, expected[row]] / total).max() < 0.000001
    assert oracle_router.topk(np.array([[2., 1., 2.]], np.float32), 1, False)[0].tolist() == [[2]]


@pytest.mark.gpu
def test_router_reproduces_the_reference_router_test(gpu):
    from mlxl3_b200 import router
    values, cases = _reference_case()
    for k, expected in cases:
        ids, scores = router.topk(values, k, True)
        assert scores.dtype == np.float32 and np.array_equal(ids, expected)
        for row in range(2):
            total = values[row, expected[row]].sum(dtype=np.float32)
            assert np.abs(scores[row] - values[row, expected[row]] / total).max() < 0.000001
    assert router.topk(np.array([[2., 1., 2.]], np.float32), 1, False)[0].tolist() == [[2]]
    for bad_k in (0, 18):
        with pytest.raises(gpu.B200Exl3Error, match="invalid router top-k"):
            router.topk(values, bad_k, True)
    with pytest.raises(gpu.B200Exl3Error, match="FP16 or FP32"):
        router.topk(np.zeros((1, 17), np.uint32), 1, True)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("rows,experts,k,normalize", [(1, 128, 8, True), (5, 256, 8, True), (3, 60, 4, False), (2, 1024, 10, True), (4, 8, 8, False)])
def test_router_matches_oracle(gpu, dtype, rows, experts, k, normalize):
    from mlxl3_b200 import router
    rng = np.random.default_rng(experts + k)
    values = (rng.standard_normal((rows, experts)) * 0.02).astype(dtype)
    values[0, : experts // 4] = values[0, 0]                       # a long run of equal values
    if experts > 16:
        values[-1, 3], values[-1, 7] = 0.0, -0.0
    got_i, got_s = router.topk(values, k, normalize)
    want_i, want_s = oracle_router.topk(values, k, normalize)
    assert np.array_equal(got_i, want_i)
    assert np.array_equal(got_s.view(np.uint16 if dtype == np.float16 else np.uint32),
                          want_s.view(np.uint16 if dtype == np.float16 else np.uint32))


@pytest.mark.gpu
def test_router_specials_and_validation(gpu):
    from mlxl3_b200 import router
    values = np.array([[0.5, 2.0, 2.0, -1.0, 0.0, -0.0, np.nan, 1.0]], np.float32)
    indices, scores = router.topk(values, 4, False)
    assert indices.tolist() == [[7, 1, 2, 6]] and np.isnan(scores[0, 3])
    with pytest.raises(gpu.B200Exl3Error, match="invalid router top-k"):
        router.topk(np.zeros((1, 4), np.float16), 5, False)
    with pytest.raises(gpu.B200Exl3Error, match="at most 1024 experts"):
        router.topk(np.zeros((1, 1025), np.float16), 2, False)
    with pytest.raises(gpu.B200Exl3Error, match="rank 2"):
        router.topk(np.zeros(4, np.float16), 2, False)


def test_oracle_softmax_rows_sum_to_one_and_keep_order():
    rng = np.random.default_rng(3)
    logits = (rng.standard_normal((4, 128)) * 2).astype(np.float16)
    p = oracle_router.softmax_precise(logits)
    assert p.dtype == np.float16 and np.abs(p.astype(np.float32).sum(axis=1) - 1).max() < 2e-3
    assert np.array_equal(np.argmax(p, axis=1), np.argmax(logits, axis=1))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("rows,experts,k", [(1, 128, 8), (256, 128, 8), (7, 60, 4), (3, 1024, 10)])
def test_softmax_router_matches_oracle(gpu, dtype, rows, experts, k):
    """The softmax may differ from the oracle's by one unit in the last place (exp and the fp32 sum order are not
    pinned); the routes must be exactly the oracle's routes on the probabilities the GPU produced."""
    from mlxl3_b200 import router
    rng = np.random.default_rng(experts + rows)
    logits = (rng.standard_normal((rows, experts)) * 1.5).astype(dtype)
    ids, scores, probs = router.softmax_topk(logits, k, True)
    want = oracle_router.softmax_precise(logits)
    as_int = np.int32 if dtype == np.float32 else np.int16
    assert probs.dtype == dtype and np.abs(probs.view(as_int).astype(np.int64) - want.view(as_int).astype(np.int64)).max() <= (1 if dtype == np.float16 else 8)
    want_i, want_s = oracle_router.topk(probs, k, True)
    bits_t = np.uint16 if dtype == np.float16 else np.uint32
    assert np.array_equal(ids, want_i) and np.array_equal(scores.view(bits_t), want_s.view(bits_t))


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 8, 13, 256])
def test_router_gate_product(gpu, rows):
    from mlxl3_b200 import router
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, 2048)).astype(np.float16)
    w = (rng.standard_normal((128, 2048)) * 0.02).astype(np.float16)
    got, want = router.gate(x, w).astype(np.float32), oracle_router.gate(x, w).astype(np.float32)
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()
