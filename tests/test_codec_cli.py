"""The JSON-lines codec tool (mlxl3_b200.codec_cli) against the oracle, request by request, in the wire format of
the reference's `mlxl3-rs codec` (native/src/main.rs:286-427; its contract test native/tests/contracts.rs:571-615)."""
import io
import json

import numpy as np
import pytest

import oracle
from mlxl3_b200 import codec_cli
from tests.gpu_util import gpu  # noqa: F401


def run(requests):
    out = io.StringIO()
    codec_cli.main(io.StringIO("".join(json.dumps(r) + "\n" if isinstance(r, dict) else r + "\n" for r in requests)), out)
    return [json.loads(line) for line in out.getvalue().splitlines()]


def test_host_only_operations_and_error_survival():
    rng = np.random.default_rng(1)
    states = rng.integers(0, 65536, 512, dtype=np.uint16)
    answers = run([{"op": "permutation"}, {"op": "pack", "k": 3, "data": states.tolist()}, "not json",
                   {"op": "pack", "k": 9, "data": states.tolist()}, {"op": "pack", "k": 2, "data": [1, 2, 3]},
                   {"op": "nonsense"}, {"op": "pack", "mode": 7, "data": []}, {"op": "pack", "data": states.tolist()}])
    assert answers[0]["data"] == oracle.permutation().tolist()
    assert answers[1]["data"] == np.asarray(oracle.pack(states, 3)).reshape(-1).tolist()
    assert answers[2] == {"error": "invalid codec request"}
    assert answers[3] == {"error": "K must be in 1..=8, got 9"}
    assert answers[4] == {"error": "encoded length must be a multiple of 256"}
    assert answers[5] == {"error": "unknown or unavailable codec operation nonsense"}
    assert answers[6] == {"error": "invalid EXL3 codebook 7"}
    assert answers[7]["data"] == np.asarray(oracle.pack(states, 4)).reshape(-1).tolist()        # k defaults to 4


@pytest.mark.gpu
def test_device_operations(gpu):
    rng = np.random.default_rng(2)
    k, cb, n_in, cols = 3, 1, 256, 128
    packed = rng.integers(0, 65536, 2 * 16 * k, dtype=np.uint16)
    states = rng.integers(0, 65536, 300, dtype=np.uint16)
    trellis = rng.integers(0, 65536, (n_in // 16, cols // 16, 16 * k), dtype=np.uint16)
    suh = np.where(rng.random(n_in) > 0.5, -1, 1).astype(np.float16)
    svh = np.where(rng.random(cols) > 0.5, -1, 1).astype(np.float16)
    x = rng.standard_normal((2, n_in)).astype(np.float16)
    bits = lambda a: np.ascontiguousarray(a).view(np.uint16).reshape(-1).tolist()  # noqa: E731
    widths = [128, 256]
    members = [(rng.integers(0, 65536, (n_in // 16, w // 16, 16 * k), dtype=np.uint16),
                np.where(rng.random(n_in) > 0.5, -1, 1).astype(np.float16),
                np.where(rng.random(w) > 0.5, -1, 1).astype(np.float16)) for w in widths]
    answers = run([
        {"op": "unpack", "k": k, "data": packed.tolist()},
        {"op": "codebook", "mode": 2, "data": states.tolist()},
        {"op": "mlx-linear", "k": k, "mode": cb, "cols": cols, "data": bits(trellis), "suh": bits(suh), "svh": bits(svh), "x": bits(x)},
        {"op": "mlx-group", "k": k, "mode": cb, "widths": widths, "data": sum((bits(m[0]) for m in members), []),
         "suh": sum((bits(m[1]) for m in members), []), "svh": sum((bits(m[2]) for m in members), []), "x": bits(x)},
        {"op": "mlx-group", "k": k, "widths": [128], "data": [], "suh": bits(suh), "svh": [], "x": bits(x)},
        {"op": "unpack", "k": k, "data": [1, 2, 3]},
    ])
    assert answers[0]["data"] == np.asarray(oracle.unpack(packed, k)).reshape(-1).tolist()
    assert answers[1]["data"] == oracle.codebook_table(2)[states].view(np.uint16).tolist()
    want = oracle.linear_forward(trellis, k, cb, suh, svh, None, x).astype(np.float32)
    got = np.asarray(answers[2]["data"], np.uint16).view(np.float16).reshape(2, cols).astype(np.float32)
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    for (t, s_in, s_out), data in zip(members, answers[3]["data"]):
        want = oracle.linear_forward(t, k, cb, s_in, s_out, None, x).astype(np.float32)
        got = np.asarray(data, np.uint16).view(np.float16).reshape(2, -1).astype(np.float32)
        assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    assert answers[4] == {"error": "unsupported group"}
    assert answers[5] == {"error": "packed length is not a whole tile"}


@pytest.mark.gpu
def test_expert_stage_operations(gpu):
    """mlx-expert, mlx-swiglu-prepare and mlx-expert-reduce: the stages of the expert block one by one, in the wire
    format of native/src/main.rs:540-626, each against the oracle's function for that stage."""
    rng = np.random.default_rng(3)
    k, cb, n_in, hidden, experts, slots = 4, 0, 256, 128, 4, 3
    bits = lambda a: np.ascontiguousarray(a).view(np.uint16).reshape(-1).tolist()  # noqa: E731
    bank = rng.integers(0, 65536, (n_in // 16, 2 * experts * hidden // 16, 16 * k), dtype=np.uint16)
    selected = np.array([2, 0, 3], np.uint32)
    x = rng.standard_normal((slots * 2, n_in)).astype(np.float16)
    suh = np.where(rng.random((slots * 2, n_in)) > 0.5, -1, 1).astype(np.float16)
    svh = rng.uniform(0.5, 1.5, (slots * 2, hidden)).astype(np.float16)
    gu_svh = (rng.uniform(0.5, 1.5, (experts, 2, hidden)) / 16).astype(np.float16)
    down_suh = np.where(rng.random((experts, hidden)) > 0.5, -1, 1).astype(np.float16)
    state = (rng.standard_normal((slots * 2, hidden)) * 16).astype(np.float32)
    raw = rng.standard_normal((slots, 256)).astype(np.float32) * 8
    red_svh = rng.uniform(0.5, 1.5, (slots, 256)).astype(np.float16)
    beta = rng.random(slots).astype(np.float16)
    common = {"k": k, "mode": cb, "cols": hidden, "data": bits(bank), "x": bits(x), "suh": bits(suh), "selected": selected.tolist(),
              "projections_per_route": 2, "projection_stride_tiles": experts * hidden // 16}
    answers = run([
        dict(common, op="mlx-expert", return_raw=True, svh=[]),
        dict(common, op="mlx-expert", return_raw=False, svh=bits(svh)),
        {"op": "mlx-swiglu-prepare", "cols": hidden, "state": state.reshape(-1).tolist(), "suh": bits(gu_svh), "svh": bits(down_suh),
         "selected": selected.tolist()},
        {"op": "mlx-expert-reduce", "cols": 256, "state": raw.reshape(-1).tolist(), "svh": bits(red_svh), "beta": bits(beta)},
        dict(common, op="mlx-expert", projections_per_route=0),
    ])
    ht = hidden // 16
    want_raw = np.empty((slots * 2, hidden), np.float32)
    for slot, e in enumerate(selected):
        for p in range(2):
            r = slot * 2 + p
            c0 = (p * experts + int(e)) * ht
            want_raw[r] = oracle.matmul_raw(np.ascontiguousarray(bank[:, c0:c0 + ht]), k, cb, oracle.prepare(x[r:r + 1], suh[r]))[0]
    got_raw = np.asarray(answers[0]["data"]["f32"], np.float32).reshape(slots * 2, hidden)
    assert np.abs(got_raw - want_raw).max() <= 2e-4 * np.abs(want_raw).max()
    got = np.asarray(answers[1]["data"]["f16"], np.uint16).view(np.float16).reshape(slots * 2, hidden).astype(np.float32)
    want = oracle.finish(want_raw, svh, None).astype(np.float32)
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    want_xd = oracle.glu_down_input(state[0::2], state[1::2], gu_svh[selected, 0], gu_svh[selected, 1], down_suh[selected])
    got_xd = np.asarray(answers[2]["data"], np.uint16).view(np.float16).reshape(slots, hidden)
    assert np.abs(got_xd.astype(np.float32) - want_xd.astype(np.float32)).max() <= 1e-2 * np.abs(want_xd.astype(np.float32)).max()
    want_y = oracle.finish_and_reduce(raw, red_svh, beta.reshape(1, slots), slots)
    assert answers[3]["data"] == want_y.view(np.uint16).reshape(-1).tolist()           # rotations and fp16 sums are bit-exact
    assert answers[4] == {"error": "invalid projection count"}
