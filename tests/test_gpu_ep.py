"""Expert parallelism of the SwiGLU expert block on the GPU (b200exl3_moe_forward_ep).

One GPU: a context of world size 1 (the rank publishes to its own inbox) against the single-device block and the CPU
oracle, call after call (both inbox parities).  Two GPUs (skipped on a one-GPU box): two processes, each with half of
the experts; both ranks must end with the same bytes, within the block's stated bar of the oracle (max |got - oracle|
<= 1e-2 * max|oracle| per row, RMS difference below 2e-3 of the output RMS).
"""
import os
import socket

import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu  # noqa: F401
from tests.test_gpu_moe import check, make_bank, routes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,experts,top_k,k,cb", [(1, 16, 4, 4, 0), (7, 8, 2, 3, 1), (40, 12, 3, 2, 2)])
def test_world_of_one_matches_the_block(gpu, rows, experts, top_k, k, cb):
    from mlxl3_b200 import ep
    rng = np.random.default_rng(rows + experts)
    n_in, hidden = 256, 384
    bank = make_bank(rng, experts, n_in, hidden, k)
    ctx = ep.EpContext(0, 1, 256, n_in, lambda raw: [raw])
    sharded = ep.Exl3SwitchGluEp(*bank, top_k, k, cb, ctx, exact_weights=True)
    whole = gpu.Exl3SwitchGlu(*bank, top_k, k, cb, exact_weights=True)
    for call in range(3):
        x = rng.standard_normal((rows, n_in)).astype(np.float16)
        selected, scores = routes(rng, rows, experts, top_k)
        got = sharded.forward(x, selected, scores)
        check(got, oracle.switch_glu_forward(*bank, top_k, k, cb, x, selected, scores))
        gpu.set_option("moe_sorted", 0)
        try:
            check(got, whole.forward(x, selected, scores), rms=1e-3)
        finally:
            gpu.set_option("moe_sorted", 1)
        got32 = sharded.forward(x, selected, scores.astype(np.float32))
        assert got32.dtype == np.float32
        check(got32, got, rms=3e-3)
        assert ctx.status() == 0 and gpu.workspace_status(sharded._workspace) == 0
    # an id beyond the bank belongs to no rank: its slot contributes nothing and must not hang the combine ... it is
    # the caller's contract that routes name existing experts, so only in-range ids are exercised here
    with pytest.raises(gpu.B200Exl3Error, match="exceed the exchange buffers"):
        small = ep.EpContext(0, 1, 2, n_in, lambda raw: [raw])
        ep.Exl3SwitchGluEp(*bank, top_k, k, cb, small).forward(x, selected, scores)
    sharded.close(), whole.close(), ctx.close()


def _rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mlxl3_b200 as ex
        from mlxl3_b200 import ep
        ex.init(rank)
        rng = np.random.default_rng(31)
        experts, top_k, n_in, hidden, k, cb = 16, 4, 256, 256, 3, 0
        bank = make_bank(rng, experts, n_in, hidden, k)

        def exchange(raw):
            gathered = [None] * world
            dist.all_gather_object(gathered, raw)
            return gathered
        ctx = ep.EpContext(rank, world, 512, n_in, exchange)
        block = ep.Exl3SwitchGluEp(*bank, top_k, k, cb, ctx, exact_weights=True)
        results = []
        dist.barrier()
        for rows in (1, 9, 70, 1):
            x = rng.standard_normal((rows, n_in)).astype(np.float16)
            selected, scores = routes(rng, rows, experts, top_k)
            results.append((x, selected, scores, block.forward(x, selected, scores)))
        status = ctx.status()
        dist.barrier()
        out.put((rank, results, status))
        dist.barrier()
        ctx.close()
    finally:
        dist.destroy_process_group()


def test_two_gpus_share_the_experts(gpu):
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
    for _ in range(600):
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
    assert got[0][2] == 0 and got[1][2] == 0
    rng = np.random.default_rng(31)
    bank = make_bank(rng, 16, 256, 256, 3)
    for (x, selected, scores, y0), (_, _, _, y1) in zip(got[0][1], got[1][1]):
        assert np.array_equal(bits(y0), bits(y1))
        check(y0, oracle.switch_glu_forward(*bank, 4, 3, 0, x, selected, scores))
