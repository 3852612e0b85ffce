"""Times one EXL3 linear layer on the GPU: ``python -m mlxl3_b200.layer_bench --in 4096 --out 14336 --k 4 --rows 1``.

Random trellis words, unit scales, activations resident in device memory.  Prints one JSON line with
the mean time of a forward call (CUDA events around ``--iters`` calls after ``--warmup`` calls), the
packed-weight bytes per second for small batches and the multiply-add rate for large ones.  It is also
the small, fixed workload that kernel profiles are captured on.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import F16, Exl3Linear, init, new_workspace, set_option, workspace_status
from .runtime import DeviceBuffer, Event, Graph, Stream


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--in", dest="n_in", type=int, default=4096)
    ap.add_argument("--out", dest="n_out", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4, help="bits per weight (1..8)")
    ap.add_argument("--cb", type=int, default=0, help="codebook: 0 default, 1 MCG, 2 MUL1")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--exact", action="store_true", help="bit-exact fp16 weights in the small-batch kernel")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="b200exl3_set_option before the run")
    ap.add_argument("--no-graph", action="store_true", help="launch every call from the host instead of replaying a graph")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--experts", type=int, default=0,
                    help="> 0: time the grouped-expert SwiGLU block instead (--in = model width, --out = expert width)")
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--step-layers", type=int, default=0,
                    help="> 0: time the persistent decode-step kernel on this many Llama-3-8B-shaped decoder layers "
                         "([q|k|v], o, [gate|up], down at --k bits, chained), one launch per step")
    ap.add_argument("--decoder-layers", type=int, default=0,
                    help="> 0: time one decode step of a Llama-3-8B-shaped dense decoder with this many layers at --context keys")
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--unfused", action="store_true", help="with --decoder-layers: norms and SwiGLU as kernels of their own")
    ap.add_argument("--stacked", action="store_true",
                    help="with --decoder-layers: o, [gate|up], down and the next block's [q|k|v] as one persistent launch per block")
    ap.add_argument("--trace", action="store_true", help="with --step-layers: print the per-layer phase stamps of one step")
    ap.add_argument("--step-plain", action="store_true",
                    help="with --step-layers: that many plain layers of --in x --out instead of decoder blocks (chained when square)")
    args = ap.parse_args(argv)
    if args.experts > 0:
        return moe_main(args)
    if args.step_layers > 0:
        return step_main(args)
    if args.decoder_layers > 0:
        return decoder_main(args)

    init(args.device)
    for item in args.option:
        name, value = item.split("=")
        set_option(name, int(value))
    rng = np.random.default_rng(0)
    trellis = rng.integers(0, 65536, (args.n_in // 16, args.n_out // 16, 16 * args.k), dtype=np.uint16)
    layer = Exl3Linear(trellis, np.ones(args.n_in, np.float16), np.ones(args.n_out, np.float16), None, args.k, args.cb,
                       exact_weights=args.exact)
    x = rng.standard_normal((args.rows, args.n_in)).astype(np.float16)
    stream = Stream()
    d_x = DeviceBuffer.from_numpy(x, stream)
    d_y = DeviceBuffer(args.rows * args.n_out * 2)
    ws = new_workspace(layer.workspace_bytes(args.rows))
    for _ in range(args.warmup):
        layer.forward_device(d_x.ptr, F16, args.rows, d_y.ptr, ws, stream)
    stream.sync()
    start, stop = Event(), Event()
    if args.no_graph:
        start.record(stream)
        for _ in range(args.iters):
            layer.forward_device(d_x.ptr, F16, args.rows, d_y.ptr, ws, stream)
        stop.record(stream)
    else:
        # the calls are recorded once and replayed, so that host launch cost does not hide short kernels
        with Graph.record(stream) as graph:
            for _ in range(args.iters):
                layer.forward_device(d_x.ptr, F16, args.rows, d_y.ptr, ws, stream)
        graph.launch(stream)
        stream.sync()
        start.record(stream)
        graph.launch(stream)
        stop.record(stream)
    stream.sync()
    ms = start.elapsed_ms(stop) / max(args.iters, 1)
    status = workspace_status(ws)
    if status:
        raise SystemExit(f"kernel reported status {status}")
    weight_bytes = args.n_in * args.n_out * args.k / 8
    print(json.dumps({
        "in": args.n_in, "out": args.n_out, "k": args.k, "cb": args.cb, "rows": args.rows,
        "us_per_forward": round(ms * 1e3, 2),
        "weight_GBps": round(weight_bytes / ms / 1e6, 1),
        "TFLOPs": round(2.0 * args.rows * args.n_in * args.n_out / ms / 1e9, 1),
    }))


def step_main(args) -> None:
    """The decode-step kernel (``Exl3Stack``) on ``--step-layers`` decoder layers of the Llama-3-8B shape, every
    projection reading the output of the one before it."""
    from . import Exl3Group, Exl3Stack

    init(args.device)
    for item in args.option:
        name, value = item.split("=")
        set_option(name, int(value))
    rng = np.random.default_rng(0)
    hidden, ffn, kv, k = 4096, 14336, 1024, args.k

    def lin(n_in, n_out):
        trellis = rng.integers(0, 65536, (n_in // 16, n_out // 16, 16 * k), dtype=np.uint16)
        svh = np.full(n_out, 1.0 / (1.2437 * np.sqrt(n_in)), np.float16)
        return Exl3Linear(trellis, np.ones(n_in, np.float16), svh, None, k, args.cb, exact_weights=args.exact)
    stream = Stream()
    source = DeviceBuffer.from_numpy(rng.standard_normal((1, hidden)).astype(np.float16), stream)
    ops, names, keep, nbytes = [], [], [], 0
    for _ in range(args.step_layers if args.step_plain else 0):
        y = DeviceBuffer(args.n_out * 2)
        if not ops:
            source = DeviceBuffer.from_numpy(rng.standard_normal((1, args.n_in)).astype(np.float16), stream)
        ops.append((lin(args.n_in, args.n_out), source.ptr, y.ptr))
        names.append("plain")
        nbytes += args.n_in * args.n_out * k // 8
        keep += [y, source]
        if args.n_in == args.n_out:
            source = y
    for _ in range(0 if args.step_plain else args.step_layers):
        q, kk, v, o, gate, up, down = (DeviceBuffer(n * 2) for n in (hidden, kv, kv, hidden, ffn, ffn, hidden))
        ops += [(Exl3Group([lin(hidden, hidden), lin(hidden, kv), lin(hidden, kv)]), source.ptr, [q.ptr, kk.ptr, v.ptr]),
                (lin(hidden, hidden), q.ptr, o.ptr),
                (Exl3Group([lin(hidden, ffn), lin(hidden, ffn)]), o.ptr, [gate.ptr, up.ptr]),
                (lin(ffn, hidden), gate.ptr, down.ptr)]
        names += ["qkv", "o", "gate|up", "down"]
        nbytes += (hidden * (hidden + 2 * kv) + hidden * hidden + 2 * hidden * ffn + ffn * hidden) * k // 8
        keep += [q, kk, v, o, gate, up, down]
        source = down
    stack = Exl3Stack(ops, F16, 1)
    grid, smem = stack.geometry()
    for _ in range(args.warmup):
        stack.forward(stream)
    stream.sync()
    start, stop = Event(), Event()
    start.record(stream)
    for _ in range(args.iters):
        stack.forward(stream)
    stop.record(stream)
    ms = start.elapsed_ms(stop) / max(args.iters, 1)
    if stack.status():
        raise SystemExit(f"kernel reported status {stack.status()}")
    print(json.dumps({"step_layers": args.step_layers, "k": k, "grid": grid, "smem_per_cta": smem, "us_per_step": round(ms * 1e3, 2),
                      "us_per_layer": round(ms * 1e3 / args.step_layers, 2), "weight_GBps": round(nbytes / ms / 1e6, 1)}))
    if args.trace:
        slots = 8 + 12                                    # stamps per (layer, CTA): see kStackTraceSlots
        trace = DeviceBuffer(len(ops) * grid * slots * 8)
        trace.fill(0, stream)
        set_option("stack_trace_buffer", trace.ptr)
        stack.forward(stream)
        stream.sync()
        set_option("stack_trace_buffer", 0)
        t = trace.download((len(ops), grid, slots), np.uint64, stream).astype(np.float64)
        t0 = t[t > 0].min()
        end_prev = 0.0
        for i, name in enumerate(names):
            s = np.where(t[i] > 0, (t[i] - t0) / 1e3, np.nan)
            done = s[:, 8:]
            fin = s[~np.isnan(s[:, 7])]
            end = float(np.nanmax(fin[:, 7])) if len(fin) else float("nan")
            owner = s[~np.isnan(s[:, 7])]                # CTAs that finished a block of this layer (their last one)
            chain = ""
            if len(owner):
                chain = (f" | finish of a block: pieces waited {np.nanmedian(owner[:, 6] - owner[:, 4]):5.2f} (max {np.nanmax(owner[:, 6] - owner[:, 4]):5.2f}), "
                         f"rotate+store {np.nanmedian(owner[:, 7] - owner[:, 6]):5.2f}")
            print(f"{i:3d} {name:8s} start {end_prev:8.2f} | boundary passed {np.nanmin(s[:, 0]):8.2f}..{np.nanmax(s[:, 0]):8.2f} | rotated {np.nanmax(s[:, 1]):8.2f} | "
                  f"tiles done p50 {np.nanpercentile(done, 50):8.2f} max {np.nanmax(done):8.2f} | last block stored {end:8.2f} | "
                  f"layer {end - end_prev:6.2f} us{chain}")
            end_prev = end


def decoder_main(args) -> None:
    """One decode step of ``DenseDecoder`` (embedding, blocks, final norm, fp16 head, arg-max) with synthetic weights."""
    from .decoder import DecoderConfig, DenseDecoder, SyntheticWeights

    init(args.device)
    for item in args.option:
        name, value = item.split("=")
        set_option(name, int(value))
    config = DecoderConfig(layers=args.decoder_layers, k_bits=args.k, codebook=args.cb, max_ctx=args.context)
    model = DenseDecoder(config, SyntheticWeights(config, seed=1))
    model.fused = not args.unfused
    model.stacked = args.stacked
    model.fill_cache(args.context - 1)
    model.set_input(17, args.context - 1)
    if not args.no_graph:
        model.record()
    for _ in range(args.warmup):
        model.step()
    model.stream.sync()
    start, stop = Event(), Event()
    start.record(model.stream)
    for _ in range(args.iters):
        model.step()
    stop.record(model.stream)
    ms = start.elapsed_ms(stop) / max(args.iters, 1)
    value, index = model.result()
    print(json.dumps({"decoder_layers": args.decoder_layers, "context": args.context, "k": args.k, "ms_per_token": round(ms, 4),
                      "launches_per_token": model.launches_per_step, "bytes_per_token": config.bytes_per_token(args.context),
                      "GBps": round(config.bytes_per_token(args.context) / ms / 1e6, 1), "argmax": index, "finite": bool(np.isfinite(value))}))


def moe_main(args) -> None:
    """``Exl3SwitchGlu.forward`` on random banks: every token picks ``top_k`` distinct experts at random."""
    from . import Exl3SwitchGlu

    init(args.device)
    for item in args.option:
        name, value = item.split("=")
        set_option(name, int(value))
    rng = np.random.default_rng(0)
    e, n_in, hidden, k = args.experts, args.n_in, args.n_out, args.k
    gu = rng.integers(0, 65536, (n_in // 16, e * hidden // 8, 16 * k), dtype=np.uint16)
    down = rng.integers(0, 65536, (hidden // 16, e * n_in // 16, 16 * k), dtype=np.uint16)
    ones = lambda *shape: np.ones(shape, np.float16)  # noqa: E731
    block = Exl3SwitchGlu(gu, ones(e, 2, n_in), ones(e, 2, hidden) / np.float16(64), down, ones(e, hidden),
                          ones(e, n_in) / np.float16(32), args.top_k, k, args.cb, exact_weights=args.exact)
    rows = args.rows
    x = rng.standard_normal((rows, n_in)).astype(np.float16)
    selected = np.stack([rng.permutation(e)[:args.top_k] for _ in range(rows)]).astype(np.uint32)
    scores = np.full((rows, args.top_k), 1.0 / args.top_k, np.float16)
    stream = Stream()
    d_x, d_sel, d_sc = (DeviceBuffer.from_numpy(a, stream) for a in (x, selected, scores))
    d_y = DeviceBuffer(rows * n_in * 2)
    ws = new_workspace(block.workspace_bytes(rows))

    def call() -> None:
        block.forward_device(d_x.ptr, F16, rows, d_sel.ptr, d_sc.ptr, F16, d_y.ptr, ws, stream)
    for _ in range(args.warmup):
        call()
    stream.sync()
    start, stop = Event(), Event()
    if args.no_graph:
        start.record(stream)
        for _ in range(args.iters):
            call()
        stop.record(stream)
    else:
        with Graph.record(stream) as graph:
            for _ in range(args.iters):
                call()
        graph.launch(stream)
        stream.sync()
        start.record(stream)
        graph.launch(stream)
        stop.record(stream)
    stream.sync()
    ms = start.elapsed_ms(stop) / max(args.iters, 1)
    status = workspace_status(ws)
    if status:
        raise SystemExit(f"kernel reported status {status}")
    # bytes of the expert columns a call touches at least once (distinct experts), and the reads it issues
    distinct = len(np.unique(selected))
    per_expert = 3 * n_in * hidden * k / 8
    print(json.dumps({
        "experts": e, "top_k": args.top_k, "in": n_in, "hidden": hidden, "k": k, "cb": args.cb, "rows": rows,
        "us_per_forward": round(ms * 1e3, 2),
        "routed_weight_GBps": round(rows * args.top_k * per_expert / ms / 1e6, 1),
        "distinct_expert_GBps": round(distinct * per_expert / ms / 1e6, 1),
    }))


if __name__ == "__main__":
    main()
