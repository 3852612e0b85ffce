"""GPU parity of the codec kernels, through the C ABI: every result must be bit-identical."""
import json

import numpy as np
import pytest

import oracle
from tests.gpu_util import bits, gpu  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cb", range(3))
def test_codebook_all_65536_states(gpu, cb):
    got = gpu.codec.codebook(None, cb)
    assert got.size == 65536
    assert np.array_equal(bits(got), bits(oracle.codebook_table(cb)))


def test_native_quantizer_fixture(gpu, golden_dir):
    data = np.load(golden_dir / "native_quantizer.npz")
    for k in range(2, 9):
        for cb in range(3):
            states, packed = data[f"k{k}_cb{cb}_states"], data[f"k{k}_cb{cb}_packed"]
            decoded = data[f"k{k}_cb{cb}_decoded"]
            assert np.array_equal(gpu.codec.unpack(packed, k), states)
            got = gpu.codec.decode_tiles(packed, k, cb).astype(np.float32)
            assert got.size == 1024 and np.array_equal(got.view(np.uint32), decoded.view(np.uint32))
            assert np.array_equal(bits(gpu.codec.codebook(states, cb)), bits(decoded.astype(np.float16)))


def test_checkpoint_tiles(gpu, golden_dir):
    doc = json.loads((golden_dir / "checkpoint_tiles.json").read_text())
    count = 0
    for entry in doc.values():
        for tile in entry["tiles"]:
            packed = np.array(tile["packed"], np.int64).astype(np.uint16)
            assert np.array_equal(gpu.codec.unpack(packed, entry["k"]), np.array(tile["states"], np.uint16))
            got = gpu.codec.decode_tiles(packed, entry["k"], entry["mode"])
            assert np.array_equal(bits(got), np.array(tile["f16_bits"], np.uint16))
            count += 1
    assert count == 12


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", range(3))
def test_reconstruct_inner_random(gpu, k, cb):
    rng = np.random.default_rng(100 * k + cb)
    for n_in, n_out in ((128, 256), (48, 176), (16, 16)):
        trellis = rng.integers(0, 65536, (n_in // 16, n_out // 16, 16 * k), dtype=np.uint16)
        got = gpu.codec.reconstruct_inner(trellis, k, cb)
        want = oracle.reconstruct_inner(trellis, k, cb)
        assert got.shape == want.shape == (n_in, n_out)
        assert np.array_equal(bits(got), bits(want))
        assert np.array_equal(gpu.codec.unpack(trellis, k), oracle.unpack(trellis, k))


def test_reconstruct_matches_reference_python_decoder(gpu, golden_dir):
    pony = np.load(golden_dir / "ponyexl3_ref.npz")
    for k in range(1, 9):
        for cb in range(3):
            trellis = pony[f"k{k}_cb{cb}_trellis"]
            # 2 x 3 tiles: pad to a legal tile grid is not needed, reconstruct accepts multiples of 16
            got = gpu.codec.reconstruct_inner(trellis, k, cb)
            assert np.array_equal(bits(got), pony[f"k{k}_cb{cb}_inner"])


def test_reconstruct_full_size_layer(gpu):
    # the single-layer configuration: 4096 x 4096 at 4 bits per weight
    rng = np.random.default_rng(1001)
    trellis = rng.integers(0, 65536, (256, 256, 64), dtype=np.uint16)
    got = gpu.codec.reconstruct_inner(trellis, 4, 0)
    want = oracle.reconstruct_inner(trellis, 4, 0)
    assert np.isfinite(got.astype(np.float32)).all()
    assert np.array_equal(bits(got), bits(want))


def test_empty_and_invalid(gpu):
    assert gpu.codec.unpack(np.empty(0, np.uint16), 3).size == 0
    assert gpu.codec.codebook(np.empty(0, np.uint16), 1).size == 0
    with pytest.raises(gpu.B200Exl3Error, match="not a whole tile"):
        gpu.codec.unpack(np.zeros(17, np.uint16), 1)
    with pytest.raises(gpu.B200Exl3Error, match="K must be in 1..=8"):
        gpu.codec.unpack(np.zeros(16, np.uint16), 0)
