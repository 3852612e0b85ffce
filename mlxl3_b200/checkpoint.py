"""Reader of EXL3 checkpoints on disk: safetensors shards plus ``config.json`` and ``quantization_config.json``.

Mirror of the reference's ``native/src/checkpoint.rs`` (``read_header`` :38-93, ``inspect`` :196-341) with
the same checks and error wording, so that a model directory the reference accepts can be handed to
``Exl3Linear.from_checkpoint`` / ``Exl3SwitchGlu.from_checkpoint`` unchanged.  Tensors are returned as
read-only numpy views of memory-mapped shards; nothing is copied until a layer uploads them.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

from ._lib import B200Exl3Error

_DTYPE_SIZE = {"BOOL": 1, "U8": 1, "I8": 1, "F8_E4M3": 1, "F8_E5M2": 1, "U16": 2, "I16": 2, "F16": 2, "BF16": 2,
               "U32": 4, "I32": 4, "F32": 4, "U64": 8, "I64": 8, "F64": 8}
# bf16 has no numpy type: its words come back as uint16 (pass scale_dtype=BF16 on)
_NUMPY = {"BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "U16": np.uint16, "I16": np.int16, "F16": np.float16,
          "BF16": np.uint16, "U32": np.uint32, "I32": np.int32, "F32": np.float32, "U64": np.uint64, "I64": np.int64,
          "F64": np.float64, "F8_E4M3": np.uint8, "F8_E5M2": np.uint8}


@dataclass
class TensorInfo:
    dtype: str
    shape: list
    data_offsets: tuple
    file: Path
    payload_offset: int


def read_header(path) -> dict:
    """Tensor table of one safetensors file (``read_header``, native/src/checkpoint.rs:38-93): 8-byte
    little-endian header length, JSON header, then a payload that the tensors must tile exactly."""
    path = Path(path)
    file_len = path.stat().st_size
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise B200Exl3Error("missing safetensors header length")
        (header_len,) = struct.unpack("<Q", raw)
        if header_len > 100_000_000 or header_len > max(file_len - 8, 0):
            raise B200Exl3Error("invalid safetensors header length")
        try:
            entries = json.loads(f.read(header_len))
        except ValueError as error:
            raise B200Exl3Error("invalid safetensors header JSON") from error
    if not isinstance(entries, dict):
        raise B200Exl3Error("invalid safetensors header JSON")
    metadata = entries.pop("__metadata__", None)
    if metadata is not None and not (isinstance(metadata, dict) and all(isinstance(v, str) for v in metadata.values())):
        raise B200Exl3Error("invalid safetensors metadata")
    payload_offset = header_len + 8
    tensors, ranges = {}, []
    for name in sorted(entries):
        value = entries[name]
        try:
            dtype, shape = value["dtype"], [int(n) for n in value["shape"]]
            start, end = (int(n) for n in value["data_offsets"])
        except (KeyError, TypeError, ValueError) as error:
            raise B200Exl3Error(f"invalid tensor {name}") from error
        if dtype not in _DTYPE_SIZE:
            raise B200Exl3Error(f"unsupported safetensors dtype {dtype}")
        if any(n < 0 for n in shape):
            raise B200Exl3Error(f"invalid tensor {name}")
        nbytes = _DTYPE_SIZE[dtype] * int(np.prod(shape, dtype=object)) if shape else _DTYPE_SIZE[dtype]
        if not (0 <= start <= end <= file_len - payload_offset and end - start == nbytes):
            raise B200Exl3Error(f"invalid data range for tensor {name}")
        tensors[name] = TensorInfo(dtype, shape, (start, end), path, payload_offset)
        ranges.append((start, end))
    at = 0
    for start, end in sorted(ranges):
        if start != at:
            raise B200Exl3Error("safetensors payload has gaps or overlapping tensors")
        at = end
    if at != file_len - payload_offset:
        raise B200Exl3Error("unclaimed safetensors payload")
    return tensors


@dataclass
class Checkpoint:
    """What ``inspect`` learned about a model directory (``Checkpoint``, native/src/checkpoint.rs)."""
    path: Path
    model_type: str
    bits: float | None
    size_bytes: int
    modules: list
    tensors: dict
    _maps: dict = field(default_factory=dict, repr=False)

    def array(self, name: str) -> np.ndarray:
        """The tensor as a read-only numpy array over the memory-mapped shard (bf16 as uint16 words)."""
        info = self.tensors.get(name)
        if info is None:
            raise B200Exl3Error(f"missing tensor {name}")
        shard = self._maps.get(info.file)
        if shard is None:
            shard = self._maps[info.file] = np.memmap(info.file, dtype=np.uint8, mode="r")
        start, end = info.data_offsets
        raw = shard[info.payload_offset + start: info.payload_offset + end]
        return raw.view(_NUMPY[info.dtype]).reshape(info.shape)

    def scale_name(self, prefix: str, primary: str, legacy: str) -> str:
        """``{prefix}.suh`` when present, else the legacy ``{prefix}.su`` (native/src/linear.rs:500-511)."""
        key = f"{prefix}.{primary}"
        return key if key in self.tensors else f"{prefix}.{legacy}"

    def codebook(self, prefix: str) -> int:
        """2 (MUL1) when ``{prefix}.mul1`` exists, 1 (MCG) when ``{prefix}.mcg`` exists, else 0
        (native/src/linear.rs:512-518)."""
        if f"{prefix}.mul1" in self.tensors:
            return 2
        return 1 if f"{prefix}.mcg" in self.tensors else 0


def inspect(path) -> Checkpoint:
    """Validates a model directory and indexes its tensors (``inspect``, native/src/checkpoint.rs:196-341)."""
    try:
        path = Path(path).resolve(strict=True)
    except OSError as error:
        raise B200Exl3Error(f"model directory {path}") from error
    with open(path / "config.json") as f:
        config = json.load(f)
    if not isinstance(config, dict):
        raise B200Exl3Error("model config must be an object")
    with open(path / "quantization_config.json") as f:
        quant = json.load(f)
    if not isinstance(quant, dict) or quant.get("quant_method") != "exl3":
        raise B200Exl3Error("expected quant_method='exl3'")
    storage = quant.get("tensor_storage")
    if not isinstance(storage, dict):
        raise B200Exl3Error("invalid EXL3 tensor_storage")
    model_type = config.get("model_type") if isinstance(config.get("model_type"), str) else "unknown"
    tensors, size_bytes, tokenizer = {}, 0, False
    for entry in sorted(os.scandir(path), key=lambda e: e.name):
        if not entry.is_file():
            continue
        size_bytes += entry.stat().st_size
        name = entry.name
        tokenizer |= name.startswith("tokenizer") or name.endswith(".model") or name == "vocab.json"
        if name.startswith("model") and name.endswith(".safetensors"):
            for tensor, info in read_header(entry.path).items():
                if tensor in tensors:
                    raise B200Exl3Error(f"duplicate tensor {tensor}")
                tensors[tensor] = info
    if not tensors:
        raise B200Exl3Error("checkpoint has no safetensors weights")
    if not tokenizer:
        raise B200Exl3Error("missing tokenizer files; download the complete checkpoint")
    modules = []
    for prefix, metadata in storage.items():
        if not isinstance(metadata, dict):
            raise B200Exl3Error(f"invalid tensor_storage entry {prefix}")
        stored = metadata.get("stored_tensors")
        if stored is not None:
            if not isinstance(stored, dict):
                raise B200Exl3Error("invalid stored_tensors")
            for name, spec in stored.items():
                try:
                    shape = [int(n) for n in spec["shape"]]
                except (KeyError, TypeError, ValueError) as error:
                    raise B200Exl3Error("invalid stored tensor shape") from error
                info = tensors.get(name)
                if info is None:
                    raise B200Exl3Error(f"missing tensor {name}")
                if info.shape != shape:
                    raise B200Exl3Error(f"invalid shape for tensor {name}")
        if metadata.get("quant_format") != "exl3":
            continue
        t = tensors.get(f"{prefix}.trellis")
        if t is None:
            raise B200Exl3Error(f"missing trellis {prefix}")
        if not (t.dtype in ("U16", "I16") and len(t.shape) == 3 and all(n > 0 for n in t.shape)
                and t.shape[2] % 16 == 0 and t.shape[2] <= 128):
            raise B200Exl3Error(f"invalid EXL3 trellis {prefix}")
        for axis, primary, legacy in ((0, "suh", "su"), (1, "svh", "sv")):
            scale = tensors.get(f"{prefix}.{primary}") or tensors.get(f"{prefix}.{legacy}")
            if scale is None:
                raise B200Exl3Error(f"missing scale {prefix}.{primary}")
            if scale.shape != [t.shape[axis] * 16]:
                raise B200Exl3Error(f"invalid scale shape {prefix}.{primary}")
            if scale.dtype not in ("F16", "BF16", "F32"):
                raise B200Exl3Error(f"invalid scale dtype {prefix}.{primary}")
        modules.append(prefix)
    if not modules:
        raise B200Exl3Error("checkpoint contains no EXL3 modules")
    modules.sort()
    index = path / "model.safetensors.index.json"
    if index.exists():
        with open(index) as f:
            weight_map = json.load(f).get("weight_map")
        if not isinstance(weight_map, dict):
            raise B200Exl3Error("invalid shard index")
        for name, shard in weight_map.items():
            if not isinstance(shard, str):
                raise B200Exl3Error("invalid shard name")
            if Path(shard).name != shard:
                raise B200Exl3Error("invalid shard path")
            info = tensors.get(name)
            if info is None:
                raise B200Exl3Error(f"missing indexed tensor {name}")
            if info.file.name != shard:
                raise B200Exl3Error(f"tensor {name} is in the wrong shard")
    bits = quant.get("bits")
    return Checkpoint(path, model_type, float(bits) if isinstance(bits, (int, float)) else None, size_bytes, modules, tensors)


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Writes ``{name: numpy array}`` as one safetensors file (used by tests and to export synthetic layers).
    uint16 arrays named in ``metadata['bf16']`` (comma-separated) are stored as BF16."""
    names = {np.dtype(v): k for k, v in _NUMPY.items() if k not in ("BF16", "F8_E4M3", "F8_E5M2")}
    bf16 = set((metadata or {}).get("bf16", "").split(",")) - {""}
    header, payload, at = {}, [], 0
    for name in sorted(tensors):
        a = np.asarray(tensors[name])
        if not a.flags.c_contiguous:
            a = np.ascontiguousarray(a)
        raw = a.tobytes()
        header[name] = {"dtype": "BF16" if name in bf16 else names[a.dtype], "shape": list(a.shape),
                        "data_offsets": [at, at + len(raw)]}
        payload.append(raw)
        at += len(raw)
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for raw in payload:
            f.write(raw)
