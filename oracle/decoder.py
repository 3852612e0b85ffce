"""CPU restatement of the decoder-block glue around the quantized projections (TEST INFRASTRUCTURE ONLY).

What is restated: the operators a decoder block of the reference runs between its EXL3 projections, in the order of
native/src/lfm2.rs:704-793 (projections -> RoPE -> cache append -> attention -> output projection) and of the dense
MLP (gate|up -> swiglu -> down), with the residual adds and RMSNorms of a pre-norm decoder.  The reference reaches
these operators through MLX 0.32.2 (native/src/array.rs:1517-1519, 1662-1664, 1741-1743, 1766-1777;
native/ffi/mlx_bridge.cpp:678, 743, 745-750, 846-849), a third-party dependency that is not in the reference tree:
its published arithmetic is restated (fp32 inside each operator, one rounding to fp16 at its output; rms_norm rounds
the normalised value to fp16 before multiplying by the weight; rope rotates the pairs (i, i + dims/2)).

Parity status: UNPINNED for these operators -- the reference holds no stored outputs of them; comparisons against this
file use the stated tolerances of the tests.
"""
from __future__ import annotations

import numpy as np

F16 = np.float16


def rms_norm(x, weight, eps, residual=None):
    """Returns (y, s): s = half(x + residual) (or x), y = weight * half(s * rsqrt(mean(s^2) + eps))."""
    s = np.asarray(x, F16)
    if residual is not None:
        s = (s.astype(np.float32) + np.asarray(residual, F16).astype(np.float32)).astype(F16)
    f = s.astype(np.float32)
    inv = 1.0 / np.sqrt((f * f).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
    normed = (f * inv.astype(np.float32)).astype(F16)
    return (np.asarray(weight, F16).astype(np.float32) * normed.astype(np.float32)).astype(F16), s


def swiglu(gate, up):
    g = np.asarray(gate, F16).astype(np.float32)
    s = (1.0 / (1.0 + np.exp(-g, dtype=np.float32))).astype(F16)
    t = (g * s.astype(np.float32)).astype(F16)
    return (t.astype(np.float32) * np.asarray(up, F16).astype(np.float32)).astype(F16)


def rope(x, pos, theta):
    """x [heads, dim] fp16 -> rotated fp16; pairs (i, i + dim/2), angle pos * theta^(-2i/dim)."""
    x = np.asarray(x, F16).astype(np.float32)
    dim = x.shape[-1]
    i = np.arange(dim // 2, dtype=np.float32)
    inv_freq = np.exp2(-np.log2(np.float32(theta)) * (2 * i) / np.float32(dim)).astype(np.float32)
    ang = (np.float32(pos) * inv_freq).astype(np.float32)
    cs, sn = np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)
    a, b = x[..., : dim // 2], x[..., dim // 2:]
    return np.concatenate([a * cs - b * sn, a * sn + b * cs], axis=-1).astype(F16)


def attention_decode(q, keys, values, scale):
    """q [heads, dim]; keys, values [kv_heads, n, dim] (fp16) -> [heads, dim] fp16; softmax in fp32."""
    q = np.asarray(q, F16).astype(np.float32)
    k = np.asarray(keys, F16).astype(np.float32)
    v = np.asarray(values, F16).astype(np.float32)
    heads, kv_heads = q.shape[0], k.shape[0]
    group = heads // kv_heads
    out = np.empty_like(q)
    for h in range(heads):
        s = (k[h // group] @ q[h]) * np.float32(scale)
        p = np.exp(s - s.max(), dtype=np.float32)
        out[h] = (p @ v[h // group]) / p.sum(dtype=np.float32)
    return out.astype(F16)


def head_argmax(x, weight):
    """fp16 logits (fp32 accumulation) and the first index of their maximum."""
    logits = (np.asarray(weight, F16).astype(np.float32) @ np.asarray(x, F16).astype(np.float32).reshape(-1)).astype(F16)
    return logits, int(np.argmax(logits))


def dense_decoder_step(model: dict, token: int, pos: int, k_cache, v_cache, linear):
    """One decode step of a pre-norm dense decoder.  `model` holds numpy weights: embed, head, final_norm, theta, eps,
    heads, kv_heads, head_dim and a list `layers` of dicts with attn_norm, mlp_norm and the projections q, k, v, o,
    gate, up, down (each whatever `linear(projection, x)` accepts).  k_cache / v_cache: per layer [kv_heads, ctx, dim]
    fp16 arrays, updated in place at row `pos`.  Returns (logits, argmax, hidden_out)."""
    heads, kv_heads, dim = model["heads"], model["kv_heads"], model["head_dim"]
    h = np.asarray(model["embed"][token], F16)[None, :]
    pending = None
    for li, layer in enumerate(model["layers"]):
        xn, h = rms_norm(h, layer["attn_norm"], model["eps"], pending)
        q = rope(linear(layer["q"], xn).reshape(heads, dim), pos, model["theta"])
        k = rope(linear(layer["k"], xn).reshape(kv_heads, dim), pos, model["theta"])
        v = linear(layer["v"], xn).reshape(kv_heads, dim)
        k_cache[li][:, pos], v_cache[li][:, pos] = k, v
        att = attention_decode(q, k_cache[li][:, : pos + 1], v_cache[li][:, : pos + 1], dim ** -0.5)
        o = linear(layer["o"], att.reshape(1, heads * dim))
        xn, h = rms_norm(h, layer["mlp_norm"], model["eps"], o)
        act = swiglu(linear(layer["gate"], xn), linear(layer["up"], xn))
        pending = linear(layer["down"], act)
    xn, h = rms_norm(h, model["final_norm"], model["eps"], pending)
    logits, best = head_argmax(xn, model["head"])
    return logits, best, h
