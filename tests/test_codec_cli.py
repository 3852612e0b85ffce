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
