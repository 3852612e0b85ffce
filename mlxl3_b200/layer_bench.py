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
    args = ap.parse_args(argv)

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


if __name__ == "__main__":
    main()
