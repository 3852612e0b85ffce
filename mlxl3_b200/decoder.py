"""Decoder-block glue and a dense pre-norm decoder for batch-1 decode over the C ABI.

``ops`` functions are thin device-pointer wrappers of the glue entry points (``b200exl3_rms_norm`` ...), the
counterparts of the array operators the reference's decoder blocks call between their EXL3 projections
(native/src/lfm2.rs:704-793).  ``DenseDecoder`` strings them together with ``Exl3Linear`` / ``Exl3Group`` projections
into a Llama-shaped model (RMSNorm, RoPE, grouped-query attention over an fp16 KV cache, SwiGLU MLP, fp16 embedding
and head) with column/row tensor parallelism; one decode step is recorded once and replayed as a graph.
"""
from __future__ import annotations

from ctypes import byref, c_float, c_int64, c_size_t, c_void_p
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import F16
from .linear import Exl3Group, Exl3Linear, Prologue, new_workspace
from .runtime import DEFAULT_STREAM, DeviceBuffer, Graph, Stream


def _p(x):
    return c_void_p(x) if x else None


def embed(d_table: int, d_tokens: int, rows: int, vocab: int, hidden: int, d_out: int, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_embed", _p(d_table), _p(d_tokens), rows, vocab, hidden, _p(d_out), _p(stream.handle))


def rms_norm(d_x: int, d_residual: int, d_weight: int, rows: int, n: int, eps: float, d_sum: int, d_y: int,
             stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_rms_norm", _p(d_x), _p(d_residual), _p(d_weight), rows, n, c_float(eps), _p(d_sum), _p(d_y), _p(stream.handle))


def swiglu(d_gate: int, d_up: int, n: int, d_out: int, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_swiglu", _p(d_gate), _p(d_up), n, _p(d_out), _p(stream.handle))


def rope_append(d_q: int, d_k: int, d_v: int, heads: int, kv_heads: int, head_dim: int, d_pos: int, theta: float, max_ctx: int,
                d_k_cache: int, d_v_cache: int, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_rope_append", _p(d_q), _p(d_k), _p(d_v), heads, kv_heads, head_dim, _p(d_pos), c_float(theta), max_ctx,
              _p(d_k_cache), _p(d_v_cache), _p(stream.handle))


def attention_workspace_bytes(heads: int, kv_heads: int) -> int:
    out = c_size_t()
    _lib.call("b200exl3_attention_workspace_bytes", heads, kv_heads, byref(out))
    return out.value


def new_attention_workspace(heads: int, kv_heads: int) -> DeviceBuffer:
    """Scratch of ``attention_decode``: it starts with arrival counters that must be zero before the first call."""
    ws = DeviceBuffer(attention_workspace_bytes(heads, kv_heads))
    ws.fill(0)
    return ws


def attention_decode(d_q: int, d_k_cache: int, d_v_cache: int, heads: int, kv_heads: int, head_dim: int, d_pos: int, max_ctx: int,
                     scale: float, d_out: int, workspace: DeviceBuffer, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_attention_decode", _p(d_q), _p(d_k_cache), _p(d_v_cache), heads, kv_heads, head_dim, _p(d_pos), max_ctx,
              c_float(scale), _p(d_out), _p(workspace.ptr), workspace.nbytes, _p(stream.handle))


def head_workspace_bytes() -> int:
    out = c_size_t()
    _lib.call("b200exl3_head_workspace_bytes", byref(out))
    return out.value


def head_argmax(d_x: int, d_weight: int, vocab: int, hidden: int, index_offset: int, d_logits: int, d_best_value: int,
                d_best_index: int, workspace: DeviceBuffer, stream: Stream = DEFAULT_STREAM) -> None:
    _lib.call("b200exl3_head_argmax", _p(d_x), _p(d_weight), vocab, hidden, c_int64(index_offset), _p(d_logits), _p(d_best_value),
              _p(d_best_index), _p(workspace.ptr), workspace.nbytes, _p(stream.handle))


@dataclass
class DecoderConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    k_bits: int = 4
    codebook: int = 0
    theta: float = 500000.0
    eps: float = 1e-5
    max_ctx: int = 2048

    def bytes_per_token(self, context: int) -> int:
        """Algorithmic bytes one decode step must read: packed projection weights with their sign vectors, the
        fp16 head, and the keys and values of `context` tokens."""
        def proj(n_in, n_out):
            return n_in * n_out * self.k_bits // 8 + 2 * (n_in + n_out) + 2 * (n_in + n_out)
        kv = self.kv_heads * self.head_dim
        per_layer = (proj(self.hidden, self.heads * self.head_dim) + 2 * proj(self.hidden, kv) + proj(self.heads * self.head_dim, self.hidden)
                     + 2 * proj(self.hidden, self.ffn) + proj(self.ffn, self.hidden) + 2 * kv * context * 2)
        return self.layers * per_layer + self.vocab * self.hidden * 2


class SyntheticWeights:
    """Seeded random weights of a dense decoder, produced layer by layer (a full-size model is several GB): uniform
    random trellis words (any bit string is a valid EXL3 tile), +-1 input signs, output scales +-c with
    c = 1 / (1.2437 * sqrt(in)) so that activations keep a magnitude of about one (1.2437 is the standard deviation of
    the default codebook's values), norm weights near one, fp16 embedding ~ N(0, 1) and head ~ N(0, 1/hidden)."""

    NAMES = ("q", "k", "v", "o", "gate", "up", "down")

    def __init__(self, config: DecoderConfig, seed: int = 0):
        self.config, self.seed = config, seed

    def shape(self, name: str) -> tuple[int, int]:
        c = self.config
        qd, kvd = c.heads * c.head_dim, c.kv_heads * c.head_dim
        return {"q": (c.hidden, qd), "k": (c.hidden, kvd), "v": (c.hidden, kvd), "o": (qd, c.hidden),
                "gate": (c.hidden, c.ffn), "up": (c.hidden, c.ffn), "down": (c.ffn, c.hidden)}[name]

    def projection(self, layer: int, name: str):
        n_in, n_out = self.shape(name)
        rng = np.random.default_rng([self.seed, 1, layer, self.NAMES.index(name)])
        trellis = rng.integers(0, 65536, (n_in // 16, n_out // 16, 16 * self.config.k_bits), dtype=np.uint16)
        suh = np.where(rng.random(n_in) > 0.5, -1, 1).astype(np.float16)
        scale = np.float16(1.0 / (1.2437 * np.sqrt(n_in)))
        svh = (np.where(rng.random(n_out) > 0.5, -1, 1).astype(np.float16) * scale).astype(np.float16)
        return trellis, suh, svh

    def norm(self, layer: int, which: int) -> np.ndarray:
        rng = np.random.default_rng([self.seed, 2, layer, which])
        return (1.0 + 0.1 * rng.standard_normal(self.config.hidden)).astype(np.float16)

    def embed(self) -> np.ndarray:
        rng = np.random.default_rng([self.seed, 3])
        return rng.standard_normal((self.config.vocab, self.config.hidden), dtype=np.float32).astype(np.float16)

    def head(self) -> np.ndarray:
        rng = np.random.default_rng([self.seed, 4])
        c = self.config
        return (rng.standard_normal((c.vocab, c.hidden), dtype=np.float32) / np.float32(np.sqrt(c.hidden))).astype(np.float16)


class DenseDecoder:
    """A dense pre-norm decoder resident on one GPU (one rank of a tensor-parallel group): per layer RMSNorm ->
    [q|k|v] -> RoPE + cache append -> grouped-query attention -> o (+ residual) -> RMSNorm -> [gate|up] -> SwiGLU ->
    down (+ residual); then the final norm, the fp16 head and its arg-max.  Column-parallel projections keep this
    rank's heads / FFN columns, row-parallel ones (o, down) add the ranks' partial sums inside their kernel through
    ``tp`` (a ``TpContext``); the head is sharded over the vocabulary.  ``step()`` runs one token; after ``record()``
    it replays a recorded graph."""

    def __init__(self, config: DecoderConfig, weights, rank: int = 0, world: int = 1, tp=None, stream: Stream | None = None):
        from . import tp as tp_rules
        c = config
        if c.heads % world or c.kv_heads % world or c.ffn % (128 * world) or c.vocab % world:
            raise _lib.B200Exl3Error(f"the model does not split over {world} ranks")
        self.config, self.rank, self.world, self.tp = c, rank, world, tp
        self.stream = stream or Stream()
        self.heads, self.kv_heads, self.ffn = c.heads // world, c.kv_heads // world, c.ffn // world
        self.vocab = c.vocab // world
        self.layers = []

        def make(layer: int, name: str, kind: str) -> Exl3Linear:
            trellis, suh, svh = weights.projection(layer, name)
            if world > 1 and kind == "col":
                trellis, suh, svh, _ = tp_rules.column_shard(trellis, suh, svh, None, rank, world)
            elif world > 1:
                (trellis, suh, svh, _), _ = tp_rules.row_shard(trellis, suh, svh, None, rank, world)
            return Exl3Linear(trellis, suh, svh, None, c.k_bits, c.codebook)
        for layer in range(c.layers):
            q, k, v = (make(layer, n, "col") for n in ("q", "k", "v"))
            gate, up = (make(layer, n, "col") for n in ("gate", "up"))
            entry = {"qkv": Exl3Group([q, k, v]), "o": make(layer, "o", "row"), "gu": Exl3Group([gate, up]), "down": make(layer, "down", "row"),
                     "attn_norm": DeviceBuffer.from_numpy(weights.norm(layer, 0)), "mlp_norm": DeviceBuffer.from_numpy(weights.norm(layer, 1)),
                     "k_cache": DeviceBuffer(self.kv_heads * c.max_ctx * c.head_dim * 2), "v_cache": DeviceBuffer(self.kv_heads * c.max_ctx * c.head_dim * 2)}
            for m in (q, k, v, gate, up):
                m.close()
            self.layers.append(entry)
        self.final_norm = DeviceBuffer.from_numpy(weights.norm(c.layers, 0))
        self.embed_table = DeviceBuffer.from_numpy(weights.embed())
        self.head_weight = DeviceBuffer.from_numpy(np.ascontiguousarray(weights.head()[rank * self.vocab:(rank + 1) * self.vocab]))
        qd, kvd = self.heads * c.head_dim, self.kv_heads * c.head_dim
        self.buf = {name: DeviceBuffer(n * 2) for name, n in (("h", c.hidden), ("xn", c.hidden), ("q", qd), ("k", kvd), ("v", kvd), ("att", qd),
                                                               ("o", c.hidden), ("gate", self.ffn), ("up", self.ffn), ("act", self.ffn),
                                                               ("down", c.hidden), ("logits", self.vocab), ("h2", c.hidden))}
        self.d_token, self.d_pos = DeviceBuffer(16), DeviceBuffer(16)
        self.sumsq = DeviceBuffer(max(c.hidden // 128, 4) * 4)      # sums of squares of the residual row per 128-block
        self.d_best_value, self.d_best_index = DeviceBuffer(16), DeviceBuffer(16)
        ops = [e[n] for e in self.layers for n in ("qkv", "o", "gu", "down")]
        self.ws = new_workspace(max(op.workspace_bytes(1) for op in ops))
        self.attn_ws = new_attention_workspace(self.heads, self.kv_heads)
        self.head_ws = DeviceBuffer(head_workspace_bytes())
        self.graph = None
        self.store_logits = False
        self.fused = True            # norms, residual adds and SwiGLU run inside the projections' kernels; False: as kernels of their own
        self.stacked = False         # True (with fused, one GPU): o, [gate|up], down and the next block's [q|k|v] are ONE persistent launch
        self.stacks = None
        self.hidden_name = "h"       # buffer that holds the residual stream after a step
        self.launches_per_step = 0

    def set_input(self, token: int, pos: int) -> None:
        self.d_token.upload(np.array([token], np.int32), self.stream)
        self.d_pos.upload(np.array([pos], np.int32), self.stream)

    def fill_cache(self, tokens: int, seed: int = 0) -> None:
        """Synthetic context: rows 0..tokens-1 of every cache get random fp16 values ~ N(0, 1)."""
        c = self.config
        rng = np.random.default_rng([seed, 5, self.rank])
        for e in self.layers:
            for name in ("k_cache", "v_cache"):
                block = np.zeros((self.kv_heads, c.max_ctx, c.head_dim), np.float16)
                block[:, :tokens] = rng.standard_normal((self.kv_heads, tokens, c.head_dim), dtype=np.float32).astype(np.float16)
                e[name].upload(block, self.stream)
        self.stream.sync()

    def _row(self, op, d_x: int, d_y: int) -> None:
        if self.tp is not None:
            self.tp.forward(op, d_x, F16, 1, d_y, self.ws, self.stream)
        else:
            op.forward_device(d_x, F16, 1, d_y, self.ws, self.stream)

    def _build_stacks(self) -> None:
        """One decode-step object per block: o (+ residual), [gate|up] (RMSNorm from block sums), down (SwiGLU, + residual)
        and the NEXT block's [q|k|v] (RMSNorm from block sums, rotary embedding, cache append)."""
        from .stack import Exl3Stack
        c, b = self.config, self.buf
        h, sq = b["h"].ptr, self.sumsq.ptr
        self.stacks = []
        for l, e in enumerate(self.layers):
            ops = [(e["o"], b["att"].ptr, 0, self.tp, Prologue.plain().with_residual(h, h, sq)),
                   (e["gu"], h, [b["gate"].ptr, b["up"].ptr], None, Prologue.rms_norm_from_blocks(e["mlp_norm"].ptr, c.eps, sq)),
                   (e["down"], b["gate"].ptr, 0, self.tp, Prologue.swiglu(b["up"].ptr).with_residual(h, h, sq))]
            if l + 1 < len(self.layers):
                n = self.layers[l + 1]
                ops.append((n["qkv"], h, [b["q"].ptr, 0, 0], None,
                            Prologue.rms_norm_from_blocks(n["attn_norm"].ptr, c.eps, sq).with_rope(self.d_pos.ptr, c.theta, c.max_ctx,
                                                                                                   n["k_cache"].ptr, n["v_cache"].ptr)))
            self.stacks.append(Exl3Stack(ops, F16, 1))

    def _launch_stacked(self) -> None:
        c, b, s = self.config, self.buf, self.stream
        if self.stacks is None:
            self._build_stacks()
        h = b["h"].ptr
        embed(self.embed_table.ptr, self.d_token.ptr, 1, c.vocab, c.hidden, h, s)
        e0 = self.layers[0]
        e0["qkv"].forward_fused_device(Prologue.rms_norm(e0["attn_norm"].ptr, c.eps).with_rope(self.d_pos.ptr, c.theta, c.max_ctx, e0["k_cache"].ptr,
                                                                                             e0["v_cache"].ptr), h, 1, [b["q"].ptr, 0, 0], self.ws, s)
        for e, stack in zip(self.layers, self.stacks):
            attention_decode(b["q"].ptr, e["k_cache"].ptr, e["v_cache"].ptr, self.heads, self.kv_heads, c.head_dim, self.d_pos.ptr, c.max_ctx,
                             c.head_dim ** -0.5, b["att"].ptr, self.attn_ws, s)
            stack.forward(s)
        rms_norm(h, 0, self.final_norm.ptr, 1, c.hidden, c.eps, 0, b["xn"].ptr, s)
        self.hidden_name = "h"
        head_argmax(b["xn"].ptr, self.head_weight.ptr, self.vocab, c.hidden, self.rank * self.vocab, b["logits"].ptr if self.store_logits else 0,
                    self.d_best_value.ptr, self.d_best_index.ptr, self.head_ws, s)
        self.launches_per_step = 2 * len(self.layers) + 5

    def _launch(self) -> None:
        # one persistent launch per block: single GPU only (with tensor parallelism the per-layer kernels run)
        if self.fused and self.stacked and self.config.head_dim == 128 and self.tp is None:
            return self._launch_stacked()
        if self.fused:
            return self._launch_fused()
        c, b, s = self.config, self.buf, self.stream
        count = 0
        embed(self.embed_table.ptr, self.d_token.ptr, 1, c.vocab, c.hidden, b["h"].ptr, s)
        pending = 0
        for e in self.layers:
            rms_norm(b["h"].ptr, pending, e["attn_norm"].ptr, 1, c.hidden, c.eps, b["h"].ptr if pending else 0, b["xn"].ptr, s)
            e["qkv"].forward_device(b["xn"].ptr, F16, 1, [b["q"].ptr, b["k"].ptr, b["v"].ptr], self.ws, s)
            rope_append(b["q"].ptr, b["k"].ptr, b["v"].ptr, self.heads, self.kv_heads, c.head_dim, self.d_pos.ptr, c.theta, c.max_ctx,
                        e["k_cache"].ptr, e["v_cache"].ptr, s)
            attention_decode(b["q"].ptr, e["k_cache"].ptr, e["v_cache"].ptr, self.heads, self.kv_heads, c.head_dim, self.d_pos.ptr, c.max_ctx,
                             c.head_dim ** -0.5, b["att"].ptr, self.attn_ws, s)
            self._row(e["o"], b["att"].ptr, b["o"].ptr)
            rms_norm(b["h"].ptr, b["o"].ptr, e["mlp_norm"].ptr, 1, c.hidden, c.eps, b["h"].ptr, b["xn"].ptr, s)
            e["gu"].forward_device(b["xn"].ptr, F16, 1, [b["gate"].ptr, b["up"].ptr], self.ws, s)
            swiglu(b["gate"].ptr, b["up"].ptr, self.ffn, b["act"].ptr, s)
            self._row(e["down"], b["act"].ptr, b["down"].ptr)
            pending = b["down"].ptr
            count += 9
        rms_norm(b["h"].ptr, pending, self.final_norm.ptr, 1, c.hidden, c.eps, b["h"].ptr, b["xn"].ptr, s)
        head_argmax(b["xn"].ptr, self.head_weight.ptr, self.vocab, c.hidden, self.rank * self.vocab, b["logits"].ptr if self.store_logits else 0,
                    self.d_best_value.ptr, self.d_best_index.ptr, self.head_ws, s)
        self.launches_per_step = count + 4

    def _launch_fused(self) -> None:
        """The same step with the glue folded into the projections' kernels: the residual add runs in the epilogue of
        o and down (which hold every output block in registers) and leaves the sum of squares of each 128-block, the
        RMSNorm of the next projection is its input-rotation prologue (it only adds those block sums), and SwiGLU is the
        prologue of down, the rotary embedding and the cache append are the epilogue of [q|k|v], and the attention merges its
        splits itself.  5 launches per block instead of 10."""
        c, b, s = self.config, self.buf, self.stream
        h, sq = b["h"].ptr, self.sumsq.ptr
        embed(self.embed_table.ptr, self.d_token.ptr, 1, c.vocab, c.hidden, h, s)
        first = True
        for e in self.layers:
            pro = Prologue.rms_norm(e["attn_norm"].ptr, c.eps) if first else Prologue.rms_norm_from_blocks(e["attn_norm"].ptr, c.eps, sq)
            first = False
            if c.head_dim == 128:
                # rotary embedding and cache append in the kernel that produces q, k and v
                e["qkv"].forward_fused_device(pro.with_rope(self.d_pos.ptr, c.theta, c.max_ctx, e["k_cache"].ptr, e["v_cache"].ptr), h, 1,
                                              [b["q"].ptr, b["k"].ptr, b["v"].ptr], self.ws, s)
            else:
                e["qkv"].forward_fused_device(pro, h, 1, [b["q"].ptr, b["k"].ptr, b["v"].ptr], self.ws, s)
                rope_append(b["q"].ptr, b["k"].ptr, b["v"].ptr, self.heads, self.kv_heads, c.head_dim, self.d_pos.ptr, c.theta, c.max_ctx,
                            e["k_cache"].ptr, e["v_cache"].ptr, s)
            attention_decode(b["q"].ptr, e["k_cache"].ptr, e["v_cache"].ptr, self.heads, self.kv_heads, c.head_dim, self.d_pos.ptr, c.max_ctx,
                             c.head_dim ** -0.5, b["att"].ptr, self.attn_ws, s)
            e["o"].forward_fused_device(Prologue.plain().with_residual(h, h, sq), b["att"].ptr, 1, 0, self.ws, s, tp=self.tp)
            e["gu"].forward_fused_device(Prologue.rms_norm_from_blocks(e["mlp_norm"].ptr, c.eps, sq), h, 1, [b["gate"].ptr, b["up"].ptr],
                                         self.ws, s)
            e["down"].forward_fused_device(Prologue.swiglu(b["up"].ptr).with_residual(h, h, sq), b["gate"].ptr, 1, 0, self.ws, s, tp=self.tp)
        rms_norm(h, 0, self.final_norm.ptr, 1, c.hidden, c.eps, 0, b["xn"].ptr, s)
        self.hidden_name = "h"
        head_argmax(b["xn"].ptr, self.head_weight.ptr, self.vocab, c.hidden, self.rank * self.vocab, b["logits"].ptr if self.store_logits else 0,
                    self.d_best_value.ptr, self.d_best_index.ptr, self.head_ws, s)
        self.launches_per_step = (5 if c.head_dim == 128 else 7) * len(self.layers) + 4

    def record(self) -> None:
        self._launch()                                  # every distinct call once before recording
        self.stream.sync()
        with Graph.record(self.stream) as graph:
            self._launch()
        self.graph = graph

    def step(self) -> None:
        if self.graph is not None:
            self.graph.launch(self.stream)
        else:
            self._launch()

    def result(self) -> tuple[float, int]:
        """This rank's best (logit, vocabulary index); with several ranks the caller keeps the largest (lowest index on ties)."""
        value = self.d_best_value.download((1,), np.float32, self.stream)
        index = self.d_best_index.download((1,), np.int64, self.stream)
        return float(value[0]), int(index[0])

    def download(self, name: str) -> np.ndarray:
        return self.buf[name].download((self.buf[name].nbytes // 2,), np.float16, self.stream)


class DenseMlp:
    """The dense SwiGLU MLP block for any number of rows: [gate|up] as one ``Exl3Group``, SwiGLU, down.  With 9 rows
    and more every projection runs on the tensor cores (tcgen05); below that on the fused small-batch kernel."""

    def __init__(self, gate: Exl3Linear, up: Exl3Linear, down: Exl3Linear):
        if gate.cols != up.cols or down.rows != gate.cols or down.cols != gate.rows:
            raise _lib.B200Exl3Error("MLP projections disagree")
        self.group, self.down = Exl3Group([gate, up]), down
        self.hidden, self.ffn = gate.rows, gate.cols
        self._rows, self._bufs, self._ws = 0, None, None

    def _ensure(self, rows: int) -> None:
        if rows > self._rows:
            self._bufs = [DeviceBuffer(rows * self.ffn * 2) for _ in range(2)]
            self._ws = new_workspace(max(self.group.workspace_bytes(rows), self.down.workspace_bytes(rows)))
            self._rows = rows

    def forward_device(self, d_x: int, rows: int, d_y: int, stream: Stream = DEFAULT_STREAM) -> None:
        """fp16 rows in, fp16 rows out, no host copies."""
        self._ensure(rows)
        gate, up = self._bufs
        self.group.forward_device(d_x, F16, rows, [gate.ptr, up.ptr], self._ws, stream)
        # SwiGLU is the prologue of the down projection's input rotation (any number of rows)
        self.down.forward_fused_device(Prologue.swiglu(up.ptr), gate.ptr, rows, d_y, self._ws, stream)

    def forward(self, x: np.ndarray, stream: Stream = DEFAULT_STREAM) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float16)
        rows = x.shape[0]
        d_x, d_y = DeviceBuffer.from_numpy(x, stream), DeviceBuffer(rows * self.hidden * 2)
        self.forward_device(d_x.ptr, rows, d_y.ptr, stream)
        return d_y.download((rows, self.hidden), np.float16, stream)

    def flops(self, rows: int) -> int:
        return 3 * 2 * rows * self.hidden * self.ffn
