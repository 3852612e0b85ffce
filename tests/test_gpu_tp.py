"""Row-parallel layers over peer memory (b200exl3_linear_finish_tp).

One GPU: a context of world size 1 (the rank exchanges with itself) must reproduce the plain output
rotation bit for bit, call after call.  Two GPUs (skipped when there is only one): two processes, one per
GPU, each with half of the input rows of a layer; both must end with the same bits, equal to the oracle's
sum of the two partial products rotated once, and column shards must concatenate to the full output.
"""
import os
import socket

import numpy as np
import pytest

import oracle
from tests.gpu_util import gpu  # noqa: F401

pytestmark = pytest.mark.gpu

N_IN, N_OUT, K, CB = 512, 512, 4, 0


def _layer(rows):
    rng = np.random.default_rng(404)
    trellis = rng.integers(0, 65536, (N_IN // 16, N_OUT // 16, 16 * K), dtype=np.uint16)
    suh = rng.uniform(0.5, 1.5, N_IN).astype(np.float16)
    svh = rng.uniform(0.5, 1.5, N_OUT).astype(np.float16)
    bias = (rng.standard_normal(N_OUT) * 0.1).astype(np.float16)
    x = rng.standard_normal((rows, N_IN)).astype(np.float16)
    return trellis, suh, svh, bias, x


def test_world_of_one_equals_plain_finish(gpu):
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    from mlxl3_b200.tp import TpContext
    rows = 5
    trellis, suh, svh, bias, x = _layer(rows)
    layer = gpu.Exl3Linear(trellis, suh, svh, bias, K, CB, exact_weights=True)
    stream = Stream()
    ctx = TpContext(0, 1, rows * N_OUT // 128, lambda raw: [raw])
    d_x = DeviceBuffer.from_numpy(x)
    d_yhat = DeviceBuffer(rows * N_OUT * 4)
    d_y, d_ref = DeviceBuffer(rows * N_OUT * 2), DeviceBuffer(rows * N_OUT * 2)
    ws = gpu.new_workspace(layer.workspace_bytes(rows))
    layer.forward_partial_device(d_x.ptr, gpu.F16, rows, d_yhat.ptr, ws, stream)
    layer.finish_device(d_yhat.ptr, rows, gpu.F16, d_ref.ptr, stream)
    want = d_ref.download((rows, N_OUT), np.float16, stream)
    for _ in range(3):                                   # both slots of every unit get used
        d_y.fill(0, stream)
        ctx.finish(layer, d_yhat.ptr, rows, gpu.F16, d_y.ptr, stream)
        got = d_y.download((rows, N_OUT), np.float16, stream)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # the fused form (exchange inside the layer kernel) gives the same bits as the plain forward
    layer.forward_device(d_x.ptr, gpu.F16, rows, d_ref.ptr, ws, stream)
    want = d_ref.download((rows, N_OUT), np.float16, stream)
    for _ in range(3):
        d_y.fill(0, stream)
        ctx.forward(layer, d_x.ptr, gpu.F16, rows, d_y.ptr, ws, stream)
        got = d_y.download((rows, N_OUT), np.float16, stream)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert gpu.workspace_status(ws) == 0
    assert ctx.status() == 0
    with pytest.raises(gpu.B200Exl3Error, match="exceed the exchange buffers"):
        small = TpContext(0, 1, 2, lambda raw: [raw])
        small.finish(layer, d_yhat.ptr, rows, gpu.F16, d_y.ptr, stream)
    ctx.close()
    layer.close()


def _rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mlxl3_b200 as ex
        from mlxl3_b200 import tp
        from mlxl3_b200.runtime import DeviceBuffer, Stream
        ex.init(rank)
        rows = 3
        trellis, suh, svh, bias, x = _layer(rows)

        def exchange(raw):
            gathered = [None] * world
            dist.all_gather_object(gathered, raw)
            return gathered
        ctx = tp.TpContext(rank, world, rows * N_OUT // 128, exchange)
        stream = Stream()
        (t, s_in, s_out, b), cols = tp.row_shard(trellis, suh, svh, bias, rank, world)
        layer = ex.Exl3Linear(t, s_in, s_out, b, K, CB, exact_weights=True)
        d_x = DeviceBuffer.from_numpy(np.ascontiguousarray(x[:, cols]))
        d_yhat, d_y = DeviceBuffer(rows * N_OUT * 4), DeviceBuffer(rows * N_OUT * 2)
        ws = ex.new_workspace(layer.workspace_bytes(rows))
        results = []
        dist.barrier()
        for _ in range(3):
            layer.forward_partial_device(d_x.ptr, ex.F16, rows, d_yhat.ptr, ws, stream)
            ctx.finish(layer, d_yhat.ptr, rows, ex.F16, d_y.ptr, stream)
            results.append(d_y.download((rows, N_OUT), np.float16, stream))
        partial = d_yhat.download((rows, N_OUT), np.float32, stream)
        for _ in range(3):                               # the same layer with the exchange inside its kernel
            d_y.fill(0, stream)
            ctx.forward(layer, d_x.ptr, ex.F16, rows, d_y.ptr, ws, stream)
            results.append(d_y.download((rows, N_OUT), np.float16, stream))
        # column-parallel shard of the same layer: no exchange
        tc, c_in, c_out, cb_ = tp.column_shard(trellis, suh, svh, bias, rank, world)
        col_layer = ex.Exl3Linear(tc, c_in, c_out, cb_, K, CB, exact_weights=True)
        y_col = col_layer.forward(x)
        status = ctx.status()
        dist.barrier()
        out.put((rank, results, partial, y_col, status))
        dist.barrier()
        ctx.close()
    finally:
        dist.destroy_process_group()


def test_two_gpus_row_and_column_shards(gpu):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    import queue
    got = []
    for _ in range(600):                                 # a child that raised must not leave the parent waiting
        try:
            got.append(out.get(timeout=0.5))
        except queue.Empty:
            assert all(p.exitcode in (None, 0) for p in procs), "a rank failed"
        if len(got) == 2:
            break
    assert len(got) == 2, "ranks did not report"
    got.sort(key=lambda item: item[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, res0, part0, col0, st0), (_, res1, part1, col1, st1) = got
    assert st0 == 0 and st1 == 0
    trellis, suh, svh, bias, x = _layer(3)
    # both ranks hold the same bits, on every call: rank-ordered fp32 sum, then one rotation
    want = oracle.finish(part0 + part1, svh, bias)
    for a, b in zip(res0, res1):
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
        assert np.array_equal(a.view(np.uint16), want.view(np.uint16))
    full = oracle.linear_forward(trellis, K, CB, suh, svh, bias, x).astype(np.float32)
    assert np.abs(res0[0].astype(np.float32) - full).max() <= 1e-2 * np.abs(full).max()
    y_col = np.concatenate([col0, col1], axis=1).astype(np.float32)
    assert np.abs(y_col - full).max() <= 1e-2 * np.abs(full).max()


def test_wait_that_runs_out_sets_status_and_returns(gpu):
    """Failure made on the host: a world of two on one GPU whose second rank does not exist, so its words never
    arrive.  With the wait limit shortened to 30 ms the kernel must return (nothing hangs or faults), the context's
    status must read 4, a second call must return at once, a reset must make the context clean again, and other
    work on the device must be unaffected."""
    import ctypes
    import time
    from ctypes import byref, c_int, c_void_p

    from mlxl3_b200 import _lib
    from mlxl3_b200.runtime import DeviceBuffer, Stream
    rows = 2
    trellis, suh, svh, bias, x = _layer(rows)
    layer = gpu.Exl3Linear(trellis, suh, svh, bias, K, CB, exact_weights=True)
    units = rows * N_OUT // 128
    bufs, handle = [], ctypes.create_string_buffer(64)
    for _ in range(2):
        p = c_void_p()
        _lib.call("b200exl3_tp_alloc", 2, units, byref(p), handle)
        bufs.append(p.value)
    ctx = c_void_p()
    _lib.call("b200exl3_tp_create", 0, 2, units, (c_void_p * 2)(*bufs), byref(ctx))
    stream = Stream()
    d_x, d_y, d_ref = DeviceBuffer.from_numpy(x), DeviceBuffer(rows * N_OUT * 2), DeviceBuffer(rows * N_OUT * 2)
    ws = gpu.new_workspace(layer.workspace_bytes(rows))
    gpu.set_option("tp_wait_ms", 30)
    try:
        status = c_int(-1)
        for call in range(2):
            t0 = time.perf_counter()
            _lib.call("b200exl3_linear_forward_tp", c_void_p(layer.handle), ctx, c_void_p(d_x.ptr), gpu.F16, rows,
                      c_void_p(d_y.ptr), c_void_p(ws.ptr), ws.nbytes, c_void_p(stream.handle))
            stream.sync()
            elapsed = time.perf_counter() - t0
            assert elapsed < 2.0, elapsed                    # the first call waits about 30 ms per unit at most
            _lib.call("b200exl3_tp_status", ctx, byref(status))
            assert status.value == 4
        assert gpu.workspace_status(ws) == 0                 # the layer's own copies were fine
        _lib.call("b200exl3_tp_reset", ctx)
        _lib.call("b200exl3_tp_status", ctx, byref(status))
        assert status.value == 0
        # the device and the layer are still usable: a plain forward gives the oracle's result
        layer.forward_device(d_x.ptr, gpu.F16, rows, d_ref.ptr, ws, stream)
        got = d_ref.download((rows, N_OUT), np.float16, stream).astype(np.float32)
        want = oracle.linear_forward(trellis, K, CB, suh, svh, bias, x).astype(np.float32)
        assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    finally:
        gpu.set_option("tp_wait_ms", 4000)
        _lib.load().b200exl3_tp_free(ctx)
        for p in bufs:
            _lib.call("b200exl3_free", c_void_p(p))
        layer.close()
