"""CPU restatement of the reference's stable router top-k (test infrastructure only).

Follows native/shaders/router_topk.h:1-34 (`mlxl3_rank_row`): the key of expert t is its value mapped to an
order-preserving unsigned integer (both zeros equal, NaN above everything) with t in the low bits; an expert with
`above` larger keys goes to slot k-1-above; scores are the selected values, optionally divided by their sum,
which is added in slot order in the values' own type.  Pinned by the reference's own router test
(native/src/router.rs:427-466), whose inputs and expectations tests/test_router.py restates.
"""
import numpy as np


def topk(values: np.ndarray, k: int, normalize: bool):
    values = np.asarray(values)
    dtype = values.dtype
    rows, experts = values.shape
    indices = np.empty((rows, k), np.uint32)
    scores = np.empty((rows, k), dtype)
    for r in range(rows):
        v = values[r].astype(np.float32)
        bits = np.where(v == 0.0, np.uint32(0), v.view(np.uint32)).astype(np.uint32)
        sign = (bits.view(np.int32) >> 31).view(np.uint32) | np.uint32(0x80000000)
        mono = np.where(np.isnan(v), np.uint32(0xFFFFFFFF), bits ^ sign).astype(np.uint64)
        keys = (mono << np.uint64(32)) | np.arange(experts, dtype=np.uint64)
        order = np.argsort(keys)                       # ascending keys; keys are unique
        chosen = order[-k:]
        indices[r] = chosen
        selected = values[r][chosen]
        if normalize:
            total = dtype.type(0)
            for s in selected:
                total = dtype.type(s + total)
            with np.errstate(divide="ignore", invalid="ignore"):
                scores[r] = (selected / total).astype(dtype)
        else:
            scores[r] = selected
    return indices, scores


def softmax_precise(logits: np.ndarray) -> np.ndarray:
    """Row softmax in fp32, rounded to the logits' dtype: ``exp(x - max) * (1 / sum)`` -- the arithmetic of MLX's
    ``softmax(..., precise=True)`` (third-party, MLX 0.32.2, reached through native/src/array.rs:1589).  The order
    of its fp32 sum and the last bits of its ``exp`` are not pinned by any stored reference output (parity unpinned
    for those bits); comparisons against this function allow one unit in the last place of the result."""
    logits = np.asarray(logits)
    x = logits.astype(np.float32)
    e = np.exp(x - x.max(axis=1, keepdims=True), dtype=np.float32)
    inv = np.float32(1.0) / e.sum(axis=1, keepdims=True, dtype=np.float32)
    return (e * inv).astype(logits.dtype)


def gate(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """fp16 logits of the router gate: fp32 product of fp16 operands, rounded once."""
    return (np.asarray(x, np.float16).astype(np.float32) @ np.asarray(weight, np.float16).astype(np.float32).T).astype(np.float16)
