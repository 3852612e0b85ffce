"""Expert parallelism on two CPU ranks (gloo): the dispatch plan and the combine arithmetic of mlxl3_b200.ep, computed
with the oracle's per-slot pieces, must reproduce the single-device block bit for bit -- each slot is computed by the
rank that owns its expert, the slot results are exchanged, and every rank adds them in slot order."""
import os
import socket

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mlxl3_b200 import ep

EXPERTS, TOP_K, N_IN, HIDDEN, K, CB, ROWS = 8, 3, 256, 128, 3, 1, 5


def _case():
    rng = np.random.default_rng(808)
    gu_t = rng.integers(0, 65536, (N_IN // 16, EXPERTS * HIDDEN // 8, 16 * K), dtype=np.uint16)
    down_t = rng.integers(0, 65536, (HIDDEN // 16, EXPERTS * N_IN // 16, 16 * K), dtype=np.uint16)
    sign = lambda *shape: np.where(rng.random(shape) > 0.5, -1, 1).astype(np.float16)  # noqa: E731
    gu_svh = (sign(EXPERTS, 2, HIDDEN).astype(np.float32) / np.sqrt(N_IN)).astype(np.float16)
    down_svh = (sign(EXPERTS, N_IN).astype(np.float32) / np.sqrt(HIDDEN)).astype(np.float16)
    bank = (gu_t, sign(EXPERTS, 2, N_IN), gu_svh, down_t, sign(EXPERTS, HIDDEN), down_svh)
    x = rng.standard_normal((ROWS, N_IN)).astype(np.float16)
    selected = np.stack([rng.permutation(EXPERTS)[:TOP_K] for _ in range(ROWS)]).astype(np.uint32)
    scores = rng.random((ROWS, TOP_K)).astype(np.float16)
    return bank, x, selected, scores


def _slot_result(local_bank, local_expert, x_row):
    """half(H128(half(raw down product))) * down_svh of one slot, from the rank's own banks (moe.rs:184-236, 438-533, 602-606)."""
    gu_t, gu_suh, gu_svh, down_t, down_suh, down_svh = local_bank
    per = gu_suh.shape[0]
    ht, it = HIDDEN // 16, N_IN // 16
    raw = []
    for p in range(2):
        xhat = oracle.prepare(x_row, gu_suh[local_expert, p])
        c0 = (p * per + local_expert) * ht
        raw.append(oracle.matmul_raw(np.ascontiguousarray(gu_t[:, c0:c0 + ht]), K, CB, xhat))
    xd = oracle.glu_down_input(raw[0], raw[1], gu_svh[local_expert, 0][None], gu_svh[local_expert, 1][None], down_suh[local_expert][None])
    down_raw = oracle.matmul_raw(np.ascontiguousarray(down_t[:, local_expert * it:(local_expert + 1) * it]), K, CB, xd)
    return oracle.finish(down_raw, down_svh[local_expert], None)[0]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bank, x, selected, scores = _case()
        local_bank = ep.shard_bank(*bank, rank, world)
        slots, local_experts = ep.local_plan(selected, rank, world, EXPERTS)          # dispatch
        mine = {int(s): _slot_result(local_bank, int(e), x[int(s) // TOP_K][None]) for s, e in zip(slots, local_experts)}
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)                                          # combine: every rank gets every slot
        results = {}
        for part in everyone:
            assert not set(results) & set(part)                                         # a slot has exactly one owner
            results.update(part)
        y = np.empty((ROWS, N_IN), np.float16)
        for row in range(ROWS):
            acc = None
            for t in range(TOP_K):
                v = (results[row * TOP_K + t].astype(np.float16) * scores[row, t]).astype(np.float16)
                acc = v if acc is None else (acc + v).astype(np.float16)
            y[row] = acc
        out.put((rank, y, sorted(mine)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_dispatch_and_combine_reproduce_the_block():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([out.get(timeout=120) for _ in range(2)], key=lambda item: item[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    bank, x, selected, scores = _case()
    want = oracle.switch_glu_forward(*bank, TOP_K, K, CB, x, selected, scores)
    for rank, y, slots in got:
        assert np.array_equal(y.view(np.uint16), want.view(np.uint16))
    assert sorted(got[0][2] + got[1][2]) == list(range(ROWS * TOP_K))
    owners = ep.owner_of(selected, 2, EXPERTS).reshape(-1)
    assert [int(s) for s in np.nonzero(owners == 0)[0]] == got[0][2]


def test_expert_ranges_and_bank_shards():
    assert ep.expert_range(3, 8, 128) == (48, 16)
    bank, _, _, _ = _case()
    local = ep.shard_bank(*bank, 1, 2)
    ht = HIDDEN // 16
    assert local[0].shape == (N_IN // 16, 2 * 4 * ht, 16 * K) and local[3].shape == (HIDDEN // 16, 4 * N_IN // 16, 16 * K)
    # gate columns of expert 4 come first in rank 1's bank, its up columns after the four local gates
    assert np.array_equal(local[0][:, :ht], bank[0][:, 4 * ht:5 * ht])
    assert np.array_equal(local[0][:, 4 * ht:5 * ht], bank[0][:, (EXPERTS + 4) * ht:(EXPERTS + 5) * ht])
    assert np.array_equal(local[1], bank[1][4:]) and np.array_equal(local[5], bank[5][4:])
