"""Tensor-parallel sharding on two CPU ranks (gloo): the shards of mlxl3_b200.tp, computed by the oracle,
recombine to the unsharded layer -- concatenation for column-parallel layers, an all-reduce of the fp32
partial sums followed by the output rotation for row-parallel ones."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mlxl3_b200 import tp

N_IN, N_OUT, K, CB, ROWS = 256, 512, 3, 1, 3


def _layer():
    rng = np.random.default_rng(2024)
    trellis = rng.integers(0, 65536, (N_IN // 16, N_OUT // 16, 16 * K), dtype=np.uint16)
    suh = rng.uniform(0.5, 1.5, N_IN).astype(np.float16)
    svh = rng.uniform(0.5, 1.5, N_OUT).astype(np.float16)
    bias = (rng.standard_normal(N_OUT) * 0.1).astype(np.float16)
    x = rng.standard_normal((ROWS, N_IN)).astype(np.float16)
    return trellis, suh, svh, bias, x


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        trellis, suh, svh, bias, x = _layer()
        # column-parallel: own columns, no exchange; gather only to compare
        t, s_in, s_out, b = tp.column_shard(trellis, suh, svh, bias, rank, world)
        y_col = torch.from_numpy(oracle.linear_forward(t, K, CB, s_in, s_out, b, x).copy())
        gathered = [torch.empty_like(y_col) for _ in range(world)]
        dist.all_gather(gathered, y_col)
        # row-parallel: partial sums over the rank's input rows, summed across ranks, then rotated
        (t, s_in, s_out, b), cols = tp.row_shard(trellis, suh, svh, bias, rank, world)
        partial = torch.from_numpy(oracle.matmul_raw(t, K, CB, oracle.prepare(np.ascontiguousarray(x[:, cols]), s_in)))
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
        y_row = oracle.finish(partial.numpy(), s_out, b)
        # the timing rule of the benchmark: the slowest rank's time is the job's time
        t_max = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
        if rank == 0:
            out.put((torch.cat(gathered, dim=1).numpy(), y_row, float(t_max.item())))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_recombine():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    y_col, y_row, t_max = out.get(timeout=90)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    trellis, suh, svh, bias, x = _layer()
    want = oracle.linear_forward(trellis, K, CB, suh, svh, bias, x)
    # column shards are exact: each 128-block of the output depends on its own columns only
    assert np.array_equal(y_col.view(np.uint16), want.view(np.uint16))
    # row shards change the fp32 summation order (two partial sums instead of one running sum)
    w = want.astype(np.float32)
    assert np.abs(y_row.astype(np.float32) - w).max() <= 1e-2 * np.abs(w).max()
    assert np.sqrt(((y_row.astype(np.float32) - w) ** 2).mean()) <= 1e-3 * np.sqrt((w ** 2).mean())
    assert t_max == 2.0


def test_shard_dims_rules():
    assert tp.shard_dims("col", 4096, 14336, 8) == (4096, 1792)
    assert tp.shard_dims("row", 14336, 4096, 8) == (1792, 4096)
    assert tp.shard_dims("row", 4096, 4096, 1) == (4096, 4096)
    with pytest.raises(ValueError, match="whole 128-blocks"):
        tp.shard_dims("col", 4096, 1024, 16)
    with pytest.raises(ValueError, match="unknown"):
        tp.shard_dims("diag", 128, 128, 2)
