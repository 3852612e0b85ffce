"""The on-disk reader (mlxl3_b200.checkpoint) against synthetic model directories: the safetensors table, the
directory checks of the reference's `inspect` (native/src/checkpoint.rs:196-341) with its error wording, and the
tensor-naming rules of `from_checkpoint` (native/src/linear.rs:454-575, native/src/moe.rs:629-807)."""
import json
import struct

import numpy as np
import pytest

import oracle
from mlxl3_b200 import B200Exl3Error, checkpoint
from tests.gpu_util import gpu  # noqa: F401

K = 3


def _layer(rng, n_in, n_out, k=K):
    return {"trellis": rng.integers(-32768, 32767, (n_in // 16, n_out // 16, 16 * k), dtype=np.int16),
            "suh": rng.uniform(0.5, 1.5, n_in).astype(np.float16) * np.where(rng.random(n_in) > 0.5, -1, 1).astype(np.float16),
            "svh": rng.uniform(0.5, 1.5, n_out).astype(np.float16)}


def make_model(tmp_path, extra=None, index=None, storage_patch=None):
    rng = np.random.default_rng(11)
    tensors = {}
    for part, value in _layer(rng, 256, 128).items():
        tensors[f"model.layers.0.q_proj.{part}"] = value
    tensors["model.layers.0.q_proj.mcg"] = np.array(1, np.int32)
    legacy = _layer(rng, 128, 256)
    tensors["model.layers.0.o_proj.trellis"] = legacy["trellis"]
    tensors["model.layers.0.o_proj.su"] = legacy["suh"].astype(np.float32)            # legacy names, fp32
    tensors["model.layers.0.o_proj.sv"] = legacy["svh"].astype(np.float32)
    tensors["model.layers.0.o_proj.bias"] = (rng.standard_normal(256) * 0.1).astype(np.float32)
    tensors["model.norm.weight"] = np.ones(256, np.float16)
    if extra:
        tensors.update(extra)
    checkpoint.write_safetensors(tmp_path / "model.safetensors", tensors, {"format": "pt"})
    storage = {"model.layers.0.q_proj": {"quant_format": "exl3"}, "model.layers.0.o_proj": {"quant_format": "exl3"},
               "model.norm": {"quant_format": "fp16", "stored_tensors": {"model.norm.weight": {"shape": [256]}}}}
    if storage_patch:
        storage.update(storage_patch)
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama"}))
    (tmp_path / "quantization_config.json").write_text(json.dumps({"quant_method": "exl3", "bits": 3.0, "tensor_storage": storage}))
    (tmp_path / "tokenizer.json").write_text("{}")
    if index is not None:
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": index}))
    return tensors


def test_inspect_indexes_a_model_directory(tmp_path):
    tensors = make_model(tmp_path, index={"model.norm.weight": "model.safetensors"})
    ck = checkpoint.inspect(tmp_path)
    assert ck.model_type == "llama" and ck.bits == 3.0
    assert ck.modules == ["model.layers.0.o_proj", "model.layers.0.q_proj"]
    assert set(ck.tensors) == set(tensors)
    for name, value in tensors.items():
        got = ck.array(name)
        assert got.dtype == value.dtype and got.shape == value.shape and np.array_equal(got, value)
    assert ck.codebook("model.layers.0.q_proj") == 1 and ck.codebook("model.layers.0.o_proj") == 0
    assert ck.scale_name("model.layers.0.o_proj", "suh", "su").endswith(".su")
    assert ck.size_bytes == sum(p.stat().st_size for p in tmp_path.iterdir())


def test_inspect_rejections(tmp_path):
    make_model(tmp_path)
    (tmp_path / "tokenizer.json").unlink()
    with pytest.raises(B200Exl3Error, match="missing tokenizer files"):
        checkpoint.inspect(tmp_path)
    (tmp_path / "tokenizer.json").write_text("{}")
    quant = json.loads((tmp_path / "quantization_config.json").read_text())
    (tmp_path / "quantization_config.json").write_text(json.dumps({**quant, "quant_method": "gptq"}))
    with pytest.raises(B200Exl3Error, match="expected quant_method='exl3'"):
        checkpoint.inspect(tmp_path)
    for patch, message in [({"model.layers.1.q_proj": {"quant_format": "exl3"}}, "missing trellis model.layers.1.q_proj"),
                           ({"model.norm": {"quant_format": "fp16", "stored_tensors": {"model.norm.weight": {"shape": [255]}}}},
                            "invalid shape for tensor model.norm.weight"),
                           ({"model.norm": {"quant_format": "fp16", "stored_tensors": {"model.norm.bias": {"shape": [256]}}}},
                            "missing tensor model.norm.bias")]:
        make_model(tmp_path, storage_patch=patch)
        with pytest.raises(B200Exl3Error, match=message):
            checkpoint.inspect(tmp_path)
    make_model(tmp_path, extra={"model.layers.0.q_proj.svh": np.ones(64, np.float16)})
    with pytest.raises(B200Exl3Error, match="invalid scale shape model.layers.0.q_proj.svh"):
        checkpoint.inspect(tmp_path)
    make_model(tmp_path, extra={"model.layers.0.q_proj.suh": np.ones(256, np.int16)})
    with pytest.raises(B200Exl3Error, match="invalid scale dtype model.layers.0.q_proj.suh"):
        checkpoint.inspect(tmp_path)
    make_model(tmp_path, index={"model.norm.weight": "model-00002.safetensors"})
    with pytest.raises(B200Exl3Error, match="is in the wrong shard"):
        checkpoint.inspect(tmp_path)
    make_model(tmp_path, index={"model.missing": "model.safetensors"})
    with pytest.raises(B200Exl3Error, match="missing indexed tensor model.missing"):
        checkpoint.inspect(tmp_path)


def test_read_header_rejects_malformed_files(tmp_path):
    def write(header: dict, payload: bytes, name="bad.safetensors"):
        blob = json.dumps(header).encode()
        (tmp_path / name).write_bytes(struct.pack("<Q", len(blob)) + blob + payload)
        return tmp_path / name
    good = {"a": {"dtype": "F16", "shape": [4], "data_offsets": [0, 8]}}
    assert checkpoint.read_header(write(good, bytes(8)))["a"].shape == [4]
    with pytest.raises(B200Exl3Error, match="unclaimed safetensors payload"):
        checkpoint.read_header(write(good, bytes(10)))
    with pytest.raises(B200Exl3Error, match="invalid data range for tensor a"):
        checkpoint.read_header(write({"a": {"dtype": "F16", "shape": [5], "data_offsets": [0, 8]}}, bytes(8)))
    with pytest.raises(B200Exl3Error, match="gaps or overlapping"):
        checkpoint.read_header(write({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]},
                                      "b": {"dtype": "U8", "shape": [4], "data_offsets": [2, 6]}}, bytes(6)))
    with pytest.raises(B200Exl3Error, match="unsupported safetensors dtype C64"):
        checkpoint.read_header(write({"a": {"dtype": "C64", "shape": [1], "data_offsets": [0, 8]}}, bytes(8)))
    (tmp_path / "short.safetensors").write_bytes(b"abc")
    with pytest.raises(B200Exl3Error, match="missing safetensors header length"):
        checkpoint.read_header(tmp_path / "short.safetensors")
    (tmp_path / "long.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(B200Exl3Error, match="invalid safetensors header length"):
        checkpoint.read_header(tmp_path / "long.safetensors")


@pytest.mark.gpu
def test_layers_from_a_checkpoint(gpu, tmp_path):
    tensors = make_model(tmp_path)
    ck = checkpoint.inspect(tmp_path)
    rng = np.random.default_rng(3)
    # q_proj: fp16 scales, MCG codebook flag
    q = gpu.Exl3Linear.from_checkpoint(ck, "model.layers.0.q_proj", exact_weights=True)
    assert (q.input_dims(), q.output_dims(), q.k, q.cb) == (256, 128, K, 1)
    x = rng.standard_normal((3, 256)).astype(np.float16)
    p = "model.layers.0.q_proj"
    want = oracle.linear_forward(tensors[f"{p}.trellis"].view(np.uint16), K, 1, tensors[f"{p}.suh"], tensors[f"{p}.svh"], None, x)
    got = q.forward(x)
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 1e-2 * np.abs(want.astype(np.float32)).max()
    assert np.array_equal(q.decode().view(np.uint16), oracle.reconstruct_inner(tensors[f"{p}.trellis"].view(np.uint16), K, 1).view(np.uint16))
    # o_proj: legacy scale names in fp32, a bias (stored as fp16 by the reference), default codebook
    o = gpu.Exl3Linear.from_checkpoint(ck, "model.layers.0.o_proj", exact_weights=True)
    assert (o.input_dims(), o.output_dims(), o.cb) == (128, 256, 0)
    p = "model.layers.0.o_proj"
    x = rng.standard_normal((2, 128)).astype(np.float16)
    want = oracle.linear_forward(tensors[f"{p}.trellis"].view(np.uint16), K, 0, tensors[f"{p}.su"].astype(np.float16),
                                 tensors[f"{p}.sv"].astype(np.float16), tensors[f"{p}.bias"].astype(np.float16), x)
    got = o.forward(x)
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 1e-2 * np.abs(want.astype(np.float32)).max()


@pytest.mark.gpu
def test_expert_bank_from_a_checkpoint(gpu, tmp_path):
    rng = np.random.default_rng(21)
    experts, top_k, n_in, hidden = 4, 2, 128, 256
    extra, storage = {}, {}
    for e in range(experts):
        for projection, (a, b) in {"gate_proj": (n_in, hidden), "up_proj": (n_in, hidden), "down_proj": (hidden, n_in)}.items():
            prefix = f"model.layers.0.mlp.experts.{e}.{projection}"
            layer = _layer(rng, a, b)
            layer["svh"] = (layer["svh"].astype(np.float32) / np.sqrt(a)).astype(np.float16)
            for part, value in layer.items():
                extra[f"{prefix}.{part}"] = value
            extra[f"{prefix}.mul1"] = np.array(1, np.int32)
            storage[prefix] = {"quant_format": "exl3"}
    tensors = make_model(tmp_path, extra=extra, storage_patch=storage)
    ck = checkpoint.inspect(tmp_path)
    moe = gpu.Exl3SwitchGlu.from_checkpoint(ck, "model.layers.0.mlp.experts", experts, top_k, exact_weights=True)
    assert (moe.experts, moe.input, moe.hidden, moe.k, moe.cb) == (experts, n_in, hidden, K, 2)
    name = lambda e, proj, part: tensors[f"model.layers.0.mlp.experts.{e}.{proj}.{part}"]  # noqa: E731
    gu_t = np.concatenate([name(e, "gate_proj", "trellis") for e in range(experts)] +
                          [name(e, "up_proj", "trellis") for e in range(experts)], axis=1).view(np.uint16)
    down_t = np.concatenate([name(e, "down_proj", "trellis") for e in range(experts)], axis=1).view(np.uint16)
    pair = lambda part: np.stack([np.stack([name(e, "gate_proj", part), name(e, "up_proj", part)]) for e in range(experts)])  # noqa: E731
    single = lambda part: np.stack([name(e, "down_proj", part) for e in range(experts)])  # noqa: E731
    x = rng.standard_normal((3, n_in)).astype(np.float16)
    selected = np.array([[0, 3], [2, 1], [3, 2]], np.uint32)
    scores = np.array([[0.7, 0.3], [0.5, 0.5], [0.2, 0.8]], np.float16)
    want = oracle.switch_glu_forward(gu_t, pair("suh"), pair("svh"), down_t, single("suh"), single("svh"), top_k, K, 2,
                                     x, selected, scores).astype(np.float32)
    got = moe.forward(x, selected, scores).astype(np.float32)
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
    with pytest.raises(B200Exl3Error, match="missing expert trellis"):
        gpu.Exl3SwitchGlu.from_checkpoint(ck, "model.layers.0.mlp.experts", experts + 1, top_k)
