"""Format properties the reference checks in native/src/codec.rs:193-282, on both CPU oracles."""
import numpy as np
import pytest

import oracle
from oracle import exl3_numpy as onp


@pytest.mark.parametrize("k", range(1, 9))
def test_pack_unpack_tail_biting(k):
    states = ((np.arange(768) * 391 + 1729) & 0xFFFF).astype(np.uint16)
    packed = oracle.pack(states, k)
    decoded = oracle.unpack(packed, k)
    mask = (1 << k) - 1
    assert np.array_equal(decoded & mask, states & mask)
    assert np.array_equal(oracle.pack(decoded, k), packed)
    # any bit string is a valid tile
    rng = np.random.default_rng(k)
    raw = rng.integers(0, 65536, 5 * 16 * k, dtype=np.uint16)
    assert np.array_equal(oracle.pack(oracle.unpack(raw, k), k), raw)
    assert np.array_equal(onp.pack(onp.unpack(raw.reshape(5, -1), k), k).ravel(), raw)
    # consecutive states overlap by 16-k bits
    st = oracle.unpack(raw, k).reshape(5, 256).astype(np.uint32)
    assert np.array_equal((st[:, 1:] >> k), st[:, :-1] & (0xFFFF >> k))


def test_permutation_is_the_mma_fragment_order():
    perm = oracle.permutation()
    inv = oracle.permutation_inverse()
    assert sorted(perm.tolist()) == list(range(256))
    assert np.array_equal(inv[perm], np.arange(256))
    assert np.array_equal(perm, onp.permutation())
    for row in range(16):
        for col in range(16):
            lane = (row % 8) // 2 + (col % 8) * 4
            index = 8 * lane + 4 * (col // 8) + 2 * (row // 8) + row % 2
            assert inv[row * 16 + col] == index


@pytest.mark.parametrize("cb", range(3))
def test_codebook_exhaustive(cb):
    table = oracle.codebook_table(cb)
    assert np.isfinite(table.astype(np.float32)).all()
    assert np.array_equal(table.view(np.uint16), onp.decode_codewords(np.arange(65536), cb).view(np.uint16))
    assert float(np.abs(table.astype(np.float32)).max()) < 8.0


def test_mul1_integer_shortcuts():
    # native/src/linear.rs:3352 pairwise byte sum: same 16-bit pattern as the four-byte sum
    x = (np.arange(65536, dtype=np.uint64) * 0x83DCD12D) & 0xFFFFFFFF
    four = 0x6400 + (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24)
    pairs = (x & 0x00FF00FF) + ((x >> 8) & 0x00FF00FF)
    assert np.array_equal(four, 0x6400 + (pairs & 0xFFFF) + (pairs >> 16))


def test_c_and_numpy_agree_on_rotations():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 384)).astype(np.float16)
    suh = rng.uniform(0.5, 1.5, 384).astype(np.float16)
    assert np.array_equal(oracle.prepare(x, suh).view(np.uint16), onp.prepare(x, suh).view(np.uint16))
    yhat = (rng.standard_normal((5, 384)) * 40).astype(np.float32)
    assert np.array_equal(oracle.finish(yhat, suh).view(np.uint16), onp.finish(yhat, suh).view(np.uint16))
    x32 = rng.standard_normal((2, 128)).astype(np.float32)
    assert np.array_equal(oracle.prepare(x32, suh[:128]).view(np.uint16), onp.prepare(x32, suh[:128]).view(np.uint16))


def test_linear_forward_dtypes_and_bias():
    rng = np.random.default_rng(11)
    k, cb = 3, 1
    trellis = rng.integers(0, 65536, (8, 16, 16 * k), dtype=np.uint16)
    suh = np.where(rng.random(128) > 0.5, -1, 1).astype(np.float16)
    svh = np.where(rng.random(256) > 0.5, -1, 1).astype(np.float16)
    bias = (rng.standard_normal(256) * 0.1).astype(np.float16)
    x = rng.standard_normal((4, 128)).astype(np.float16)
    y = oracle.linear_forward(trellis, k, cb, suh, svh, None, x)
    yb = oracle.linear_forward(trellis, k, cb, suh, svh, bias, x)
    assert y.dtype == np.float16 and y.shape == (4, 256)
    assert np.array_equal(yb.view(np.uint16), (y + bias).view(np.uint16))
    y32 = oracle.linear_forward(trellis, k, cb, suh, svh, None, x.astype(np.float32))
    assert y32.dtype == np.float32 and np.array_equal(y32, y.astype(np.float32))
    # row independence: each row alone gives the same bits
    for r in range(4):
        assert np.array_equal(oracle.linear_forward(trellis, k, cb, suh, svh, None, x[r:r + 1]).view(np.uint16),
                              y[r:r + 1].view(np.uint16))
    # split-K partials sum to the full product within fp32 rounding
    xh = oracle.prepare(x, suh)
    full = oracle.matmul_raw(trellis, k, cb, xh)
    parts = oracle.matmul_raw(trellis, k, cb, xh, (0, 3)) + oracle.matmul_raw(trellis, k, cb, xh, (3, 8))
    exact = oracle.matmul_raw(trellis, k, cb, xh, f64acc=True)
    assert np.abs(full - exact).max() < 1e-4 and np.abs(parts - exact).max() < 1e-4


def test_switch_glu_oracle_reduces_to_one_expert_chain():
    """With top_k = 1 and weight 1 the grouped block equals the chain written out for that expert
    (native/src/moe.rs:905-971), and a slot's result does not depend on the other rows."""
    rng = np.random.default_rng(31)
    experts, n_in, hidden, k, cb = 3, 128, 256, 3, 1
    gu_t = rng.integers(0, 65536, (n_in // 16, experts * hidden // 8, 16 * k), dtype=np.uint16)
    down_t = rng.integers(0, 65536, (hidden // 16, experts * n_in // 16, 16 * k), dtype=np.uint16)
    sign = lambda *s: np.where(rng.random(s) > 0.5, -1, 1).astype(np.float16)  # noqa: E731
    gu_suh, down_suh = sign(experts, 2, n_in), sign(experts, hidden)
    gu_svh = (sign(experts, 2, hidden).astype(np.float32) / np.sqrt(n_in)).astype(np.float16)
    down_svh = (sign(experts, n_in).astype(np.float32) / np.sqrt(hidden)).astype(np.float16)
    x = rng.standard_normal((2, n_in)).astype(np.float16)
    selected = np.array([[2], [0]], np.uint32)
    ones = np.ones((2, 1), np.float16)
    got = oracle.switch_glu_forward(gu_t, gu_suh, gu_svh, down_t, down_suh, down_svh, 1, k, cb, x, selected, ones)
    ht, it = hidden // 16, n_in // 16
    for row, e in enumerate((2, 0)):
        xr = x[row:row + 1]
        gate = oracle.matmul_raw(np.ascontiguousarray(gu_t[:, e * ht:(e + 1) * ht]), k, cb, oracle.prepare(xr, gu_suh[e, 0]))
        up = oracle.matmul_raw(np.ascontiguousarray(gu_t[:, (experts + e) * ht:(experts + e + 1) * ht]), k, cb,
                               oracle.prepare(xr, gu_suh[e, 1]))
        xd = oracle.glu_down_input(gate, up, gu_svh[e, 0][None], gu_svh[e, 1][None], down_suh[e][None])
        down = oracle.matmul_raw(np.ascontiguousarray(down_t[:, e * it:(e + 1) * it]), k, cb, xd)
        want = oracle.finish(down, down_svh[e])          # weight 1: the plain output rotation
        assert np.array_equal(got[row].view(np.uint16), want[0].view(np.uint16))
    alone = oracle.switch_glu_forward(gu_t, gu_suh, gu_svh, down_t, down_suh, down_svh, 1, k, cb, x[1:], selected[1:], ones[1:])
    assert np.array_equal(alone.view(np.uint16), got[1:].view(np.uint16))
