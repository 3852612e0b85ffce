"""Regenerates the golden fixtures in this folder from a checkout of the reference project.

    python tests/golden/make_golden.py /path/to/reference

Needs numpy only.  What it writes:

native_quantizer.npz   the reference's 21 pack/unpack/decode cases
                       (tests/fixtures/native-quantizer/oracle-{k}-{cb}-*; used by
                       tests/quantize_fixtures.rs), one array per file.
checkpoint_tiles.json  first/middle/last tile of four real EXL3 checkpoints
                       (docs/native-coverage/baselines/exl3/*.json; used by
                       native/tests/contracts.rs:617-668): packed -> states -> fp16 bits.
h128_kat.json          SHA-256 known answers of the fp16 Hadamard-128 rotation
                       (docs/native-coverage/h128/physical.json; inputs are regenerated
                       from numpy.random.default_rng(75) exactly as
                       tests/physical_prepare128.py:16-52 draws them).
ponyexl3_ref.npz       outputs of the reference's own numpy CPU implementation
                       (apps/MLXL3Studio/Vendor/PonyExl3/ponyexl3/ref), imported and run
                       by this script: unpack, decode and reconstruct_inner for every
                       K=1..8 x codebook 0..2 on seeded random trellises, and
                       linear_forward_reconstruct on small layers.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def native_quantizer(ref: Path) -> None:
    root = ref / "tests/fixtures/native-quantizer"
    meta = json.loads((root / "reference.json").read_text())
    assert meta["status"] == "complete" and len(meta["cases"]) == 21
    arrays = {}
    for case in meta["cases"]:
        k, cb = int(case["k"]), int(case["codebook"])
        arrays[f"k{k}_cb{cb}_states"] = np.fromfile(root / f"oracle-{k}-{cb}-states.u16", "<u2")
        arrays[f"k{k}_cb{cb}_packed"] = np.fromfile(root / f"oracle-{k}-{cb}-packed.u16", "<u2")
        arrays[f"k{k}_cb{cb}_decoded"] = np.fromfile(root / f"oracle-{k}-{cb}-decoded.f32", "<f4")
    np.savez_compressed(HERE / "native_quantizer.npz", **arrays)


def checkpoint_tiles(ref: Path) -> None:
    root = ref / "docs/native-coverage/baselines/exl3"
    out = {}
    for name in ("flash", "qwen-dense", "qwen-moe", "lfm-moe"):
        d = json.loads((root / f"{name}.json").read_text())
        out[name] = {
            "checkpoint": d["checkpoint"], "tensor": d["tensor"], "k": d["k"], "mode": d["mode"],
            "tiles": [{"tile": t["tile"], "packed": t["packed"], "states": t["states"], "f16_bits": t["f16_bits"]}
                      for t in d["tiles"]],
        }
    (HERE / "checkpoint_tiles.json").write_text(json.dumps(out, separators=(",", ":")))


def h128_kat(ref: Path) -> None:
    d = json.loads((ref / "docs/native-coverage/h128/physical.json").read_text())
    assert d["status"] == "passed" and d["seed"] == 75
    (HERE / "h128_kat.json").write_text(json.dumps({"seed": 75, "cases": d["cases"]}, indent=1))


def ponyexl3(ref: Path) -> None:
    sys.path.insert(0, str(ref / "apps/MLXL3Studio/Vendor/PonyExl3"))
    from ponyexl3.ref.decode import decode_packed_trellis
    from ponyexl3.ref.forward import linear_forward_reconstruct
    from ponyexl3.ref.layer import EXL3Layer
    from ponyexl3.ref.trellis import unpack_trellis

    arrays = {}
    for k in range(1, 9):
        for cb in range(3):
            rng = np.random.default_rng(9000 + 10 * k + cb)
            trellis = rng.integers(0, 65536, (2, 3, 16 * k), dtype=np.uint16)
            arrays[f"k{k}_cb{cb}_trellis"] = trellis
            arrays[f"k{k}_cb{cb}_states"] = unpack_trellis(trellis, k)
            arrays[f"k{k}_cb{cb}_inner"] = decode_packed_trellis(trellis, k, cb).view(np.uint16)
    # Whole-layer forward of the reference's Python path (fp32 Hadamard, so only a tolerance pin).
    for k, cb, n_in, n_out, rows in ((4, 0, 256, 128, 3), (3, 1, 128, 256, 2), (2, 2, 128, 128, 1)):
        rng = np.random.default_rng(9500 + k)
        trellis = rng.integers(0, 65536, (n_in // 16, n_out // 16, 16 * k), dtype=np.uint16)
        suh = np.where(rng.random(n_in) > 0.5, -1.0, 1.0).astype(np.float16)
        svh = np.where(rng.random(n_out) > 0.5, -1.0, 1.0).astype(np.float16)
        x = rng.standard_normal((rows, n_in)).astype(np.float16)
        layer = EXL3Layer(key="golden", in_features=n_in, out_features=n_out, k=k, trellis=trellis,
                          suh=suh, svh=svh, bias=None, mcg=cb == 1, mul1=cb == 2)
        y = linear_forward_reconstruct(layer, x)
        tag = f"fwd_k{k}_cb{cb}"
        arrays[tag + "_trellis"], arrays[tag + "_suh"], arrays[tag + "_svh"] = trellis, suh, svh
        arrays[tag + "_x"], arrays[tag + "_y"] = x, np.asarray(y, np.float16)
    np.savez_compressed(HERE / "ponyexl3_ref.npz", **arrays)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    reference = Path(sys.argv[1])
    native_quantizer(reference)
    checkpoint_tiles(reference)
    h128_kat(reference)
    ponyexl3(reference)
    for f in sorted(HERE.iterdir()):
        print(f.name, f.stat().st_size)
