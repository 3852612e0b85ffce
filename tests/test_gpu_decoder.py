"""GPU parity of the decoder-block glue (RMSNorm, RoPE + cache append, grouped-query decode attention, SwiGLU, fp16 head
with arg-max) and of a small dense decoder built from it, against the CPU restatement in oracle/decoder.py.

These operators are floating point with fp32 inside and fp16 at their outputs; the reference computes them through MLX,
whose last-bit behaviour no stored output pins.  Stated bars: element-wise operators within 2 units in the last place of
fp16 (exp, sin and cos differ in their last fp32 bits between libraries); attention and the head within 2e-3 of the
row's largest magnitude; a whole decode step (two layers) within 3e-2 of the largest magnitude of the hidden state and
of the logits, with an arg-max whose oracle logit is within that bar of the oracle's maximum.
"""
import numpy as np
import pytest

import oracle
from oracle import decoder as od
from tests.gpu_util import bits, gpu  # noqa: F401

pytestmark = pytest.mark.gpu


def ulps(a, b):
    """Distance in fp16 units in the last place (on the ordered integer line)."""
    def key(x):
        u = np.ascontiguousarray(x, np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


def test_rms_norm_swiglu_rope(gpu):
    from mlxl3_b200 import decoder as dec
    from mlxl3_b200.runtime import DeviceBuffer
    rng = np.random.default_rng(1)
    n = 4096
    x = rng.standard_normal((3, n)).astype(np.float16)
    r = (rng.standard_normal((3, n)) * 0.5).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    d_x, d_r, d_w = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(r), DeviceBuffer.from_numpy(w)
    d_s, d_y = DeviceBuffer(x.nbytes), DeviceBuffer(x.nbytes)
    for residual in (None, r):
        dec.rms_norm(d_x.ptr, d_r.ptr if residual is not None else 0, d_w.ptr, 3, n, 1e-5, d_s.ptr, d_y.ptr)
        want_y, want_s = od.rms_norm(x, w, 1e-5, residual)
        assert np.array_equal(bits(d_s.download((3, n), np.float16)), bits(want_s))
        assert ulps(d_y.download((3, n), np.float16), want_y).max() <= 1
    # in place on the residual stream: sum written over x
    d_h = DeviceBuffer.from_numpy(x)
    dec.rms_norm(d_h.ptr, d_r.ptr, d_w.ptr, 3, n, 1e-5, d_h.ptr, d_y.ptr)
    assert np.array_equal(bits(d_h.download((3, n), np.float16)), bits(od.rms_norm(x, w, 1e-5, r)[1]))
    # SwiGLU
    g, u = (rng.standard_normal(14336) * 2).astype(np.float16), rng.standard_normal(14336).astype(np.float16)
    d_g, d_u, d_o = DeviceBuffer.from_numpy(g), DeviceBuffer.from_numpy(u), DeviceBuffer(g.nbytes)
    dec.swiglu(d_g.ptr, d_u.ptr, g.size, d_o.ptr)
    assert ulps(d_o.download(g.shape, np.float16), od.swiglu(g, u)).max() <= 2
    # RoPE + append
    heads, kv_heads, dim, ctx, pos, theta = 8, 2, 128, 64, 37, 500000.0
    q = rng.standard_normal((heads, dim)).astype(np.float16)
    k, v = rng.standard_normal((kv_heads, dim)).astype(np.float16), rng.standard_normal((kv_heads, dim)).astype(np.float16)
    d_q, d_k, d_v = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(k), DeviceBuffer.from_numpy(v)
    d_kc, d_vc = DeviceBuffer(kv_heads * ctx * dim * 2), DeviceBuffer(kv_heads * ctx * dim * 2)
    d_kc.fill(0), d_vc.fill(0)
    d_pos = DeviceBuffer.from_numpy(np.array([pos], np.int32))
    dec.rope_append(d_q.ptr, d_k.ptr, d_v.ptr, heads, kv_heads, dim, d_pos.ptr, theta, ctx, d_kc.ptr, d_vc.ptr)
    got_q = d_q.download((heads, dim), np.float16).astype(np.float32)
    assert np.abs(got_q - od.rope(q, pos, theta).astype(np.float32)).max() <= 4e-3
    kc, vc = d_kc.download((kv_heads, ctx, dim), np.float16), d_vc.download((kv_heads, ctx, dim), np.float16)
    assert np.abs(kc[:, pos].astype(np.float32) - od.rope(k, pos, theta).astype(np.float32)).max() <= 4e-3
    assert np.array_equal(bits(vc[:, pos]), bits(v))
    assert not kc[:, :pos].any() and not kc[:, pos + 1:].any()           # only row `pos` is written
    with pytest.raises(gpu.B200Exl3Error, match="head dimension of 128"):
        dec.rope_append(d_q.ptr, d_k.ptr, d_v.ptr, heads, kv_heads, 64, d_pos.ptr, theta, ctx, d_kc.ptr, d_vc.ptr)


@pytest.mark.parametrize("heads,kv_heads,keys,ctx", [(32, 8, 2048, 2048), (4, 4, 1, 16), (16, 2, 77, 128), (64, 8, 300, 512), (4, 1, 4096, 4096)])
def test_attention_decode(gpu, heads, kv_heads, keys, ctx):
    from mlxl3_b200 import decoder as dec
    from mlxl3_b200.runtime import DeviceBuffer
    rng = np.random.default_rng(heads + keys)
    dim = 128
    q = rng.standard_normal((heads, dim)).astype(np.float16)
    kc = np.zeros((kv_heads, ctx, dim), np.float16)
    vc = np.zeros((kv_heads, ctx, dim), np.float16)
    kc[:, :keys] = rng.standard_normal((kv_heads, keys, dim)).astype(np.float16)
    vc[:, :keys] = rng.standard_normal((kv_heads, keys, dim)).astype(np.float16)
    kc[:, keys:], vc[:, keys:] = 100.0, 100.0                         # rows past the position must not be read
    d_q, d_k, d_v = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(kc), DeviceBuffer.from_numpy(vc)
    d_o = DeviceBuffer(q.nbytes)
    d_pos = DeviceBuffer.from_numpy(np.array([keys - 1], np.int32))
    ws = dec.new_attention_workspace(heads, kv_heads)
    dec.attention_decode(d_q.ptr, d_k.ptr, d_v.ptr, heads, kv_heads, dim, d_pos.ptr, ctx, dim ** -0.5, d_o.ptr, ws)
    got = d_o.download((heads, dim), np.float16)
    want = od.attention_decode(q, kc[:, :keys], vc[:, :keys], dim ** -0.5)
    assert np.isfinite(got.astype(np.float32)).all()
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2e-3 * max(1.0, np.abs(want.astype(np.float32)).max())
    dec.attention_decode(d_q.ptr, d_k.ptr, d_v.ptr, heads, kv_heads, dim, d_pos.ptr, ctx, dim ** -0.5, d_o.ptr, ws)
    assert np.array_equal(bits(got), bits(d_o.download((heads, dim), np.float16)))         # fixed merge order


def test_head_argmax(gpu):
    from mlxl3_b200 import decoder as dec
    from mlxl3_b200.runtime import DeviceBuffer
    rng = np.random.default_rng(9)
    vocab, hidden = 16032, 4096
    x = rng.standard_normal(hidden).astype(np.float16)
    w = (rng.standard_normal((vocab, hidden)) / 64).astype(np.float16)
    w[5000] = w[123]                                                  # an exact tie: the first index wins
    d_x, d_w, d_l = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(w), DeviceBuffer(vocab * 2)
    d_bv, d_bi = DeviceBuffer(16), DeviceBuffer(16)
    ws = DeviceBuffer(dec.head_workspace_bytes())
    dec.head_argmax(d_x.ptr, d_w.ptr, vocab, hidden, 1000, d_l.ptr, d_bv.ptr, d_bi.ptr, ws)
    logits = d_l.download((vocab,), np.float16)
    want, _ = od.head_argmax(x, w)
    assert np.abs(logits.astype(np.float32) - want.astype(np.float32)).max() <= 2e-3 * np.abs(want.astype(np.float32)).max()
    assert np.array_equal(bits(logits[5000:5001]), bits(logits[123:124]))
    best = int(d_bi.download((1,), np.int64)[0]) - 1000
    assert best == int(np.argmax(logits)) and float(d_bv.download((1,), np.float32)[0]) == float(logits[best])
    # without storing the logits
    dec.head_argmax(d_x.ptr, d_w.ptr, vocab, hidden, 0, 0, d_bv.ptr, d_bi.ptr, ws)
    assert int(d_bi.download((1,), np.int64)[0]) == best


def _small():
    from mlxl3_b200.decoder import DecoderConfig, SyntheticWeights
    config = DecoderConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=1024, k_bits=4, codebook=0, max_ctx=32)
    return config, SyntheticWeights(config, seed=11)


def _oracle_model(config, weights):
    def linear(p, x):
        return oracle.linear_forward(p[0], config.k_bits, config.codebook, p[1], p[2], None, np.ascontiguousarray(x, np.float16).reshape(1, -1))
    layers = []
    for l in range(config.layers):
        layer = {n: weights.projection(l, n) for n in weights.NAMES}
        layer["attn_norm"], layer["mlp_norm"] = weights.norm(l, 0), weights.norm(l, 1)
        layers.append(layer)
    model = {"embed": weights.embed(), "head": weights.head(), "final_norm": weights.norm(config.layers, 0), "theta": config.theta,
             "eps": config.eps, "heads": config.heads, "kv_heads": config.kv_heads, "head_dim": config.head_dim, "layers": layers}
    return model, linear


def test_small_decoder_steps_match_oracle(gpu):
    from mlxl3_b200.decoder import DenseDecoder
    config, weights = _small()
    model, linear = _oracle_model(config, weights)
    dec = DenseDecoder(config, weights)
    dec.store_logits = True
    kc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    vc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    for e in dec.layers:
        e["k_cache"].fill(0, dec.stream), e["v_cache"].fill(0, dec.stream)
    tokens = [3, 700, 41, 1023, 5]
    eager = []
    for pos, token in enumerate(tokens):
        dec.set_input(token, pos)
        dec.step()
        value, index = dec.result()
        logits, hidden = dec.download("logits"), dec.download("h")
        want_logits, want_best, want_h = od.dense_decoder_step(model, token, pos, kc, vc, linear)
        bar_h = 3e-2 * np.abs(want_h.astype(np.float32)).max()
        bar_l = 3e-2 * np.abs(want_logits.astype(np.float32)).max()
        assert np.abs(hidden.astype(np.float32) - want_h.astype(np.float32).ravel()).max() <= bar_h
        assert np.abs(logits.astype(np.float32) - want_logits.astype(np.float32)).max() <= bar_l
        assert index == int(np.argmax(logits)) and value == float(logits[index])
        assert float(want_logits[want_best]) - float(want_logits[index]) <= bar_l
        eager.append((bits(logits).copy(), index))
    # the same five steps replayed from a recorded graph give the same bits
    for e in dec.layers:
        e["k_cache"].fill(0, dec.stream), e["v_cache"].fill(0, dec.stream)
    dec.set_input(tokens[0], 0)
    dec.record()
    for pos, token in enumerate(tokens):
        dec.set_input(token, pos)
        dec.step()
        _, index = dec.result()
        assert index == eager[pos][1] and np.array_equal(bits(dec.download("logits")), eager[pos][0])
    assert gpu.workspace_status(dec.ws) == 0


@pytest.mark.parametrize("rows", [3, 40])
def test_dense_mlp_block(gpu, rows):
    """[gate|up] -> SwiGLU -> down against the oracle's projections and SwiGLU, on the fused kernel (3 rows) and on
    the tensor cores (40 rows: the grouped pair runs member by member through the tcgen05 product)."""
    from mlxl3_b200.decoder import DenseMlp
    from tests.gpu_util import random_layer
    rng = np.random.default_rng(50 + rows)
    hidden, ffn, k = 512, 1024, 3
    layers = []
    for n_in, n_out in ((hidden, ffn), (hidden, ffn), (ffn, hidden)):
        t, s, v = random_layer(rng, n_in, n_out, k)
        layers.append((t, s, (v.astype(np.float32) / (1.2437 * np.sqrt(n_in))).astype(np.float16)))
    mlp = DenseMlp(*(gpu.Exl3Linear(t, s, v, None, k, 0) for t, s, v in layers))
    x = rng.standard_normal((rows, hidden)).astype(np.float16)
    got = mlp.forward(x).astype(np.float32)
    g, u = (oracle.linear_forward(t, k, 0, s, v, None, x) for t, s, v in layers[:2])
    want = oracle.linear_forward(*layers[2][:1], k, 0, layers[2][1], layers[2][2], None, od.swiglu(g, u)).astype(np.float32)
    assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    assert mlp.flops(512) == 3 * 2 * 512 * hidden * ffn


def test_fused_prologues_match_the_separate_kernels(gpu):
    """The RMSNorm (+ residual) and SwiGLU prologues fused into the layer kernel against the stand-alone kernels
    followed by the plain layer: same arithmetic, so the outputs agree to the last bits except where the norm's row sum
    (added in another order) moves 1/rms by one fp32 unit."""
    from mlxl3_b200 import Prologue, decoder as dec
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    from tests.gpu_util import random_layer
    rng = np.random.default_rng(77)
    n_in, n_out, k = 1024, 512, 4
    stream = Stream()
    members = [gpu.Exl3Linear(*random_layer(rng, n_in, w, k), None, k, 0) for w in (n_out, 256)]
    group = gpu.Exl3Group(members)
    layer = gpu.Exl3Linear(*random_layer(rng, n_in, n_out, k), None, k, 0)
    for rows in (1, 2):
        x = rng.standard_normal((rows, n_in)).astype(np.float16)
        r = (rng.standard_normal((rows, n_in)) * 0.5).astype(np.float16)
        w = (1 + 0.1 * rng.standard_normal(n_in)).astype(np.float16)
        d_x, d_r, d_w = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(r), DeviceBuffer.from_numpy(w)
        d_s, d_s2, d_xn = DeviceBuffer(x.nbytes), DeviceBuffer(x.nbytes), DeviceBuffer(x.nbytes)
        ws = gpu.new_workspace(max(group.workspace_bytes(rows), layer.workspace_bytes(rows)))
        outs = [[DeviceBuffer(rows * wd * 2) for wd in (n_out, 256)] for _ in range(2)]
        # RMSNorm with residual in front of a group
        dec.rms_norm(d_x.ptr, d_r.ptr, d_w.ptr, rows, n_in, 1e-5, d_s.ptr, d_xn.ptr, stream)
        group.forward_device(d_xn.ptr, gpu.F16, rows, [o.ptr for o in outs[0]], ws, stream)
        group.forward_fused_device(Prologue.rms_norm(d_w.ptr, 1e-5, d_r.ptr, d_s2.ptr), d_x.ptr, rows, [o.ptr for o in outs[1]], ws, stream)
        assert np.array_equal(bits(d_s.download(x.shape, np.float16, stream)), bits(d_s2.download(x.shape, np.float16, stream)))
        for a, b_, wd in zip(outs[0], outs[1], (n_out, 256)):
            ya, yb = a.download((rows, wd), np.float16, stream).astype(np.float32), b_.download((rows, wd), np.float16, stream).astype(np.float32)
            assert np.abs(ya - yb).max() <= 2e-3 * np.abs(ya).max()
        # SwiGLU in front of a plain layer
        g, u = (rng.standard_normal((rows, n_in)) * 2).astype(np.float16), rng.standard_normal((rows, n_in)).astype(np.float16)
        d_g, d_u, d_a = DeviceBuffer.from_numpy(g), DeviceBuffer.from_numpy(u), DeviceBuffer(g.nbytes)
        y0, y1 = DeviceBuffer(rows * n_out * 2), DeviceBuffer(rows * n_out * 2)
        dec.swiglu(d_g.ptr, d_u.ptr, g.size, d_a.ptr, stream)
        layer.forward_device(d_a.ptr, gpu.F16, rows, y0.ptr, ws, stream)
        layer.forward_fused_device(Prologue.swiglu(d_u.ptr), d_g.ptr, rows, y1.ptr, ws, stream)
        assert np.array_equal(bits(y0.download((rows, n_out), np.float16, stream)), bits(y1.download((rows, n_out), np.float16, stream)))
        # residual epilogue, then the norm of the next layer from the block sums it left
        hres = rng.standard_normal((rows, n_out)).astype(np.float16)
        d_h, d_sq = DeviceBuffer.from_numpy(hres), DeviceBuffer(rows * (n_out // 128) * 4)
        layer.forward_fused_device(Prologue.plain().with_residual(d_h.ptr, d_h.ptr, d_sq.ptr), d_a.ptr, rows, 0, ws, stream)
        want_sum = (hres.astype(np.float32) + y0.download((rows, n_out), np.float16, stream).astype(np.float32)).astype(np.float16)
        got_sum = d_h.download((rows, n_out), np.float16, stream)
        assert np.array_equal(bits(got_sum), bits(want_sum))
        sq = d_sq.download((rows, n_out // 128), np.float32, stream)
        want_sq = (got_sum.astype(np.float32) ** 2).reshape(rows, -1, 128).sum(axis=2)
        assert np.abs(sq - want_sq).max() <= 1e-4 * want_sq.max()
        nxt = gpu.Exl3Linear(*random_layer(rng, n_out, 256, k), None, k, 0)
        wn = (1 + 0.1 * rng.standard_normal(n_out)).astype(np.float16)
        d_wn, d_n, z0, z1 = DeviceBuffer.from_numpy(wn), DeviceBuffer(rows * n_out * 2), DeviceBuffer(rows * 256 * 2), DeviceBuffer(rows * 256 * 2)
        ws2 = gpu.new_workspace(nxt.workspace_bytes(rows))
        dec.rms_norm(d_h.ptr, 0, d_wn.ptr, rows, n_out, 1e-5, 0, d_n.ptr, stream)
        nxt.forward_device(d_n.ptr, gpu.F16, rows, z0.ptr, ws2, stream)
        nxt.forward_fused_device(Prologue.rms_norm_from_blocks(d_wn.ptr, 1e-5, d_sq.ptr), d_h.ptr, rows, z1.ptr, ws2, stream)
        za, zb = z0.download((rows, 256), np.float16, stream).astype(np.float32), z1.download((rows, 256), np.float16, stream).astype(np.float32)
        assert np.abs(za - zb).max() <= 2e-3 * np.abs(za).max()
    with pytest.raises(gpu.B200Exl3Error, match="1 to 2 rows"):
        layer.forward_fused_device(Prologue.rms_norm(d_w.ptr, 1e-5), d_x.ptr, 3, y1.ptr, ws, stream)
    # the SwiGLU prologue alone takes any number of rows: from 3 rows on the input-rotation kernel applies it (fused
    # small-batch kernel up to 8 rows, tensor-core product from 9), bit-identical to the stand-alone kernel + plain layer
    for rows in (3, 12, 70):
        g, u = (rng.standard_normal((rows, n_in)) * 2).astype(np.float16), rng.standard_normal((rows, n_in)).astype(np.float16)
        d_g, d_u, d_a = DeviceBuffer.from_numpy(g), DeviceBuffer.from_numpy(u), DeviceBuffer(g.nbytes)
        y0, y1 = DeviceBuffer(rows * n_out * 2), DeviceBuffer(rows * n_out * 2)
        ws = gpu.new_workspace(layer.workspace_bytes(rows))
        dec.swiglu(d_g.ptr, d_u.ptr, g.size, d_a.ptr, stream)
        layer.forward_device(d_a.ptr, gpu.F16, rows, y0.ptr, ws, stream)
        layer.forward_fused_device(Prologue.swiglu(d_u.ptr), d_g.ptr, rows, y1.ptr, ws, stream)
        assert np.array_equal(bits(y0.download((rows, n_out), np.float16, stream)), bits(y1.download((rows, n_out), np.float16, stream)))
        assert gpu.workspace_status(ws) == 0
    with pytest.raises(gpu.B200Exl3Error, match="over its own input"):
        layer.forward_fused_device(Prologue.rms_norm(d_w.ptr, 1e-5, d_r.ptr, d_x.ptr), d_x.ptr, 1, y1.ptr, ws, stream)


def test_small_decoder_with_glue_kernels_of_their_own(gpu):
    from mlxl3_b200.decoder import DenseDecoder
    config, weights = _small()
    model, linear = _oracle_model(config, weights)
    dec = DenseDecoder(config, weights)
    dec.store_logits, dec.fused = True, False
    kc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    vc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    for e in dec.layers:
        e["k_cache"].fill(0, dec.stream), e["v_cache"].fill(0, dec.stream)
    for pos, token in enumerate([3, 700, 41]):
        dec.set_input(token, pos)
        dec.step()
        _, index = dec.result()
        logits, hidden = dec.download("logits"), dec.download(dec.hidden_name)
        want_logits, want_best, want_h = od.dense_decoder_step(model, token, pos, kc, vc, linear)
        assert np.abs(hidden.astype(np.float32) - want_h.astype(np.float32).ravel()).max() <= 3e-2 * np.abs(want_h.astype(np.float32)).max()
        bar_l = 3e-2 * np.abs(want_logits.astype(np.float32)).max()
        assert np.abs(logits.astype(np.float32) - want_logits.astype(np.float32)).max() <= bar_l
        assert float(want_logits[want_best]) - float(want_logits[index]) <= bar_l
    assert dec.launches_per_step == 9 * config.layers + 4


def test_rotary_epilogue_matches_the_separate_kernel(gpu):
    """[q | k | v] with the rotary embedding and the cache append as the group's epilogue against the group's plain forward
    followed by rope_append: the same rounding points, so the same bits up to the last place of the fp32 rotation."""
    from mlxl3_b200 import decoder as dec
    from mlxl3_b200.linear import Prologue
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    from tests.gpu_util import random_layer
    rng = np.random.default_rng(77)
    hidden, heads, kv_heads, dim, k, max_ctx, theta = 512, 4, 2, 128, 4, 64, 500000.0
    members = [gpu.Exl3Linear(*random_layer(rng, hidden, n, k), None, k, 0) for n in (heads * dim, kv_heads * dim, kv_heads * dim)]
    group = gpu.Exl3Group(members)
    stream = Stream()
    ws = gpu.new_workspace(group.workspace_bytes(1))
    x = rng.standard_normal((1, hidden)).astype(np.float16)
    d_x = DeviceBuffer.from_numpy(x)
    for pos in (0, 5, 63):
        d_pos = DeviceBuffer.from_numpy(np.array([pos], np.int32))
        q0, k0, v0 = (DeviceBuffer(n * dim * 2) for n in (heads, kv_heads, kv_heads))
        kc0, vc0, kc1, vc1 = (DeviceBuffer(kv_heads * max_ctx * dim * 2) for _ in range(4))
        for b in (kc0, vc0, kc1, vc1):
            b.fill(0, stream)
        group.forward_device(d_x.ptr, gpu.F16, 1, [q0.ptr, k0.ptr, v0.ptr], ws, stream)
        dec.rope_append(q0.ptr, k0.ptr, v0.ptr, heads, kv_heads, dim, d_pos.ptr, theta, max_ctx, kc0.ptr, vc0.ptr, stream)
        q1 = DeviceBuffer(heads * dim * 2)
        group.forward_fused_device(Prologue.plain().with_rope(d_pos.ptr, theta, max_ctx, kc1.ptr, vc1.ptr), d_x.ptr, 1, [q1.ptr, 0, 0], ws, stream)
        want_q, got_q = q0.download((heads, dim), np.float16, stream), q1.download((heads, dim), np.float16, stream)
        assert ulps(got_q, want_q).max() <= 1
        for a, b in ((kc0, kc1), (vc0, vc1)):
            want, got = a.download((kv_heads, max_ctx, dim), np.float16, stream), b.download((kv_heads, max_ctx, dim), np.float16, stream)
            assert ulps(got, want).max() <= 1
            assert np.abs(want[:, pos]).max() > 0 and not np.any(np.delete(got, pos, axis=1))
    assert gpu.workspace_status(ws) == 0
    with pytest.raises(gpu.B200Exl3Error, match="one row"):
        group.forward_fused_device(Prologue.plain().with_rope(d_pos.ptr, theta, max_ctx, kc1.ptr, vc1.ptr), d_x.ptr, 2, [q1.ptr, 0, 0], ws, stream)
    with pytest.raises(gpu.B200Exl3Error, match="belongs to a"):
        members[0].forward_fused_device(Prologue.plain().with_rope(d_pos.ptr, theta, max_ctx, kc1.ptr, vc1.ptr), d_x.ptr, 1, q1.ptr, ws, stream)


def test_small_decoder_with_one_persistent_launch_per_block(gpu):
    """o, [gate|up], down and the next block's [q|k|v] -- with their fused norms, SwiGLU, residual adds, rotary embedding
    and cache append -- as ONE decode-step launch per block: same bar against the oracle, and step by step against the
    per-layer form (other summation order inside a projection, so not the same bits)."""
    from mlxl3_b200.decoder import DenseDecoder
    config, weights = _small()
    model, linear = _oracle_model(config, weights)
    dec, ref = DenseDecoder(config, weights), DenseDecoder(config, weights)
    dec.store_logits, dec.stacked = True, True
    ref.store_logits = True
    kc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    vc = [np.zeros((config.kv_heads, config.max_ctx, config.head_dim), np.float16) for _ in range(config.layers)]
    for d in (dec, ref):
        for e in d.layers:
            e["k_cache"].fill(0, d.stream), e["v_cache"].fill(0, d.stream)
    for pos, token in enumerate([3, 700, 41, 9]):
        for d in (dec, ref):
            d.set_input(token, pos)
            d.step()
        _, index = dec.result()
        logits, hidden = dec.download("logits"), dec.download("h")
        want_logits, want_best, want_h = od.dense_decoder_step(model, token, pos, kc, vc, linear)
        bar_l = 3e-2 * np.abs(want_logits.astype(np.float32)).max()
        assert np.abs(hidden.astype(np.float32) - want_h.astype(np.float32).ravel()).max() <= 3e-2 * np.abs(want_h.astype(np.float32)).max()
        assert np.abs(logits.astype(np.float32) - want_logits.astype(np.float32)).max() <= bar_l
        assert float(want_logits[want_best]) - float(want_logits[index]) <= bar_l
        assert np.abs(logits.astype(np.float32) - ref.download("logits").astype(np.float32)).max() <= 1e-2 * np.abs(want_logits.astype(np.float32)).max()
        for a, b in zip(dec.layers, ref.layers):          # the caches were appended by the fused epilogue
            ka = a["k_cache"].download((config.kv_heads, config.max_ctx, config.head_dim), np.float16, dec.stream)
            kb = b["k_cache"].download((config.kv_heads, config.max_ctx, config.head_dim), np.float16, ref.stream)
            assert np.abs(ka.astype(np.float32) - kb.astype(np.float32)).max() <= 2e-2 * max(1.0, np.abs(kb.astype(np.float32)).max())
    assert all(s.status() == 0 for s in dec.stacks) and dec.launches_per_step == 2 * config.layers + 5
