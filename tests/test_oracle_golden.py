"""Pins both CPU oracles (C and numpy) to the reference's own golden vectors."""
import hashlib
import json

import numpy as np
import pytest

import oracle
from oracle import exl3_numpy as onp


@pytest.fixture(scope="module")
def quantizer(golden_dir):
    return np.load(golden_dir / "native_quantizer.npz")


CASES = [(k, cb) for k in range(2, 9) for cb in range(3)]


@pytest.mark.parametrize("k,cb", CASES)
def test_native_quantizer_fixture(quantizer, k, cb):
    # tests/quantize_fixtures.rs:6-61 of the reference: pack, unpack and decode must reproduce the files.
    states = quantizer[f"k{k}_cb{cb}_states"]
    packed = quantizer[f"k{k}_cb{cb}_packed"]
    decoded = quantizer[f"k{k}_cb{cb}_decoded"]
    assert states.size == 1024 and packed.size == 4 * 16 * k and decoded.size == 1024
    assert np.isfinite(decoded).all()
    for impl_pack, impl_unpack in ((oracle.pack, oracle.unpack),
                                   (lambda s, k: onp.pack(s.reshape(-1, 256), k).ravel(),
                                    lambda p, k: onp.unpack(p.reshape(-1, 16 * k), k).ravel())):
        assert np.array_equal(impl_pack(states, k), packed)
        assert np.array_equal(impl_unpack(packed, k), states)
    want = decoded.view(np.uint32)
    got_c = oracle.codebook_table(cb)[states].astype(np.float32).view(np.uint32)
    got_np = onp.decode_codewords(states, cb).astype(np.float32).view(np.uint32)
    assert np.array_equal(got_c, want)
    assert np.array_equal(got_np, want)


def test_checkpoint_tiles(golden_dir):
    # native/tests/contracts.rs:617-668 of the reference: real checkpoint tiles, packed -> states -> fp16 bits.
    doc = json.loads((golden_dir / "checkpoint_tiles.json").read_text())
    assert set(doc) == {"flash", "qwen-dense", "qwen-moe", "lfm-moe"}
    seen = 0
    for entry in doc.values():
        k, cb = entry["k"], entry["mode"]
        for tile in entry["tiles"]:
            packed = np.array(tile["packed"], np.int64).astype(np.uint16)
            states = np.array(tile["states"], np.uint16)
            bits = np.array(tile["f16_bits"], np.uint16)
            assert packed.size == 16 * k and states.size == 256 and bits.size == 256
            assert np.array_equal(oracle.unpack(packed, k), states)
            assert np.array_equal(onp.unpack(packed, k), states)
            assert np.array_equal(oracle.codebook_table(cb)[states].view(np.uint16), bits)
            assert np.array_equal(onp.decode_codewords(states, cb).view(np.uint16), bits)
            seen += 1
    assert seen == 12


def _h128_cases():
    """Inputs of tests/physical_prepare128.py:16-52 of the reference, drawn in the same order."""
    rng = np.random.default_rng(75)
    yield "all-128-basis-rows", np.eye(128, dtype=np.float16), np.ones((1, 128), np.float16)
    for rows in (1, 3, 20):
        for width in (128, 640, 2560):
            x = rng.normal(0, 1.125, (rows, width)).astype(np.float16)
            for scale_rows in sorted({1, rows}):
                scales = rng.normal(0, 0.75, (scale_rows, width)).astype(np.float16)
                yield f"mixed-{rows}x{width}-scale-rows-{scale_rows}", x, scales
    bits = np.array([0x0000, 0x8000, 1, 0x8001, 0x3C00, 0xBC00, 0x0400, 0x8400], dtype=np.uint16)
    special = np.resize(bits, (3, 128)).view(np.float16)
    special[1] = np.float16(-0.0)
    special[2] = np.resize(bits[::-1], 128).view(np.float16)
    yield "subnormal-signed-zero", special, np.ones_like(special)


def test_h128_known_answers(golden_dir):
    kat = json.loads((golden_dir / "h128_kat.json").read_text())["cases"]
    seen = set()
    for name, x, scales in _h128_cases():
        want = kat[name]
        s = np.broadcast_to(scales, x.shape) if scales.shape[0] == x.shape[0] else scales[0]
        got_c = oracle.prepare(x, np.ascontiguousarray(s))
        got_np = onp.prepare(x, scales)
        assert got_c.size == want["values"]
        for got in (got_c, got_np):
            digest = hashlib.sha256(np.ascontiguousarray(got).view("<u2").tobytes()).hexdigest()
            assert digest == want["f16le_sha256"], name
        seen.add(name)
    assert seen == set(kat)


@pytest.fixture(scope="module")
def pony(golden_dir):
    return np.load(golden_dir / "ponyexl3_ref.npz")


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", range(3))
def test_against_reference_python_decoder(pony, k, cb):
    trellis = pony[f"k{k}_cb{cb}_trellis"]
    states = pony[f"k{k}_cb{cb}_states"]
    inner = pony[f"k{k}_cb{cb}_inner"]
    assert np.array_equal(oracle.unpack(trellis, k).reshape(states.shape), states)
    assert np.array_equal(onp.unpack(trellis, k), states)
    assert np.array_equal(oracle.reconstruct_inner(trellis, k, cb).view(np.uint16), inner)
    assert np.array_equal(onp.reconstruct_inner(trellis, k, cb).view(np.uint16), inner)


@pytest.mark.parametrize("k,cb", [(4, 0), (3, 1), (2, 2)])
def test_against_reference_python_forward(pony, k, cb):
    # The reference's Python forward uses an fp32 Hadamard without the fp16 rounding points, so this is a
    # tolerance check of orientation and conventions, not a bit pin.
    tag = f"fwd_k{k}_cb{cb}"
    trellis, suh, svh = pony[tag + "_trellis"], pony[tag + "_suh"], pony[tag + "_svh"]
    x, want = pony[tag + "_x"], pony[tag + "_y"].astype(np.float32)
    got = oracle.linear_forward(trellis, k, cb, suh, svh, None, x).astype(np.float32)
    assert got.shape == want.shape and np.isfinite(got).all()
    assert np.abs(got - want).max() <= 5e-3 * np.abs(want).max()
    got_np = onp.linear_forward(trellis, k, cb, suh, svh, x).astype(np.float32)
    assert np.abs(got_np - got).max() <= 2e-3 * np.abs(want).max()
