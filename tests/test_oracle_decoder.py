"""Properties of the CPU restatement of the decoder-block glue (oracle/decoder.py)."""
import numpy as np

from oracle import decoder as od


def test_rope_is_a_rotation_and_identity_at_position_zero():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 128)).astype(np.float16)
    assert np.array_equal(od.rope(x, 0, 500000.0).view(np.uint16), x.view(np.uint16))
    y = od.rope(x, 1234, 500000.0).astype(np.float32)
    a, b = x.astype(np.float32), y
    # the norm of every pair (i, i + 64) is kept
    assert np.abs((a[:, :64] ** 2 + a[:, 64:] ** 2) - (b[:, :64] ** 2 + b[:, 64:] ** 2)).max() < 2e-2


def test_rms_norm_and_residual():
    rng = np.random.default_rng(1)
    x, r = rng.standard_normal((2, 256)).astype(np.float16), rng.standard_normal((2, 256)).astype(np.float16)
    y, s = od.rms_norm(x, np.ones(256, np.float16), 0.0, r)
    assert np.array_equal(s.view(np.uint16), (x.astype(np.float32) + r.astype(np.float32)).astype(np.float16).view(np.uint16))
    assert np.abs((y.astype(np.float32) ** 2).mean(axis=1) - 1).max() < 5e-3


def test_attention_of_one_key_returns_its_value_and_groups_share_keys():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((4, 128)).astype(np.float16)
    k, v = rng.standard_normal((2, 1, 128)).astype(np.float16), rng.standard_normal((2, 1, 128)).astype(np.float16)
    out = od.attention_decode(q, k, v, 128 ** -0.5)
    assert np.array_equal(out[0].view(np.uint16), v[0, 0].view(np.uint16)) and np.array_equal(out[3].view(np.uint16), v[1, 0].view(np.uint16))


def test_swiglu_and_head():
    g = np.array([0.0, 20.0, -20.0, 1.0], np.float16)
    out = od.swiglu(g, np.full(4, 2.0, np.float16)).astype(np.float32)
    assert out[0] == 0 and abs(out[1] - 40) < 0.1 and abs(out[2]) < 1e-3 and abs(out[3] - 2 * 0.7311) < 2e-3
    w = np.eye(8, dtype=np.float16)
    w[5] = w[2]
    logits, best = od.head_argmax(np.array([0, 1, 3, 2, 0, 0, 0, 0], np.float16), w)
    assert best == 2 and logits[5] == logits[2]
