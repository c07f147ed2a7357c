"""Seeded synthetic weights in the reference's `ASPEN_DATA` weight-file format.

File layout (reference src/apu_file_io.c:48-432 reads it; the writer in the reference's
examples/3. custom_example/custom_net.py:114-156 documents it):

    ASPEN_DATA
    LAYER:<n>            n counts conv / connected / matmul / layernorm layers from 1
    TENSOR_TYPE:WEIGHT   (or BIAS)
    DATA_SIZE:<bytes>
    DATA_START:
    <raw little-endian fp32>DATA_END
    LAYER_END

There are no pretrained weights in this tree, so the parity and benchmark inputs are drawn from
seeded distributions: He-normal (sigma = sqrt(2/fan_in)) for CNNs, N(0, 0.02) for transformers,
biases N(0, 0.01), layernorm gain 1 + N(0, 0.02) and shift N(0, 0.02).
"""
from __future__ import annotations

import numpy as np


def make_weights(weighted_layers, seed: int, scheme: str = "he"):
    """Returns [(weight, bias)] fp32 arrays, one pair per weighted layer, in file order."""
    rng = np.random.default_rng(seed)
    out = []
    for kind, shape, fan_in in weighted_layers:
        n_out = shape[0]
        if kind == "layernorm":
            w = (1.0 + 0.02 * rng.standard_normal(shape)).astype(np.float32)
            b = (0.02 * rng.standard_normal((n_out,))).astype(np.float32)
        else:
            sigma = float(np.sqrt(2.0 / fan_in)) if scheme == "he" else 0.02
            w = (sigma * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
            b = (0.01 * rng.standard_normal((n_out,))).astype(np.float32)
        out.append((w, b))
    return out


def write_aspen_data(path: str, tensors) -> None:
    """tensors: [(weight, bias)] as returned by make_weights."""
    with open(path, "wb") as f:
        f.write(b"ASPEN_DATA\n")
        for i, (w, b) in enumerate(tensors, start=1):
            for name, arr in (("WEIGHT", w), ("BIAS", b)):
                raw = np.ascontiguousarray(arr, dtype="<f4").tobytes()
                f.write(f"LAYER:{i}\nTENSOR_TYPE:{name}\nDATA_SIZE:{len(raw)}\nDATA_START:\n".encode())
                f.write(raw)
                f.write(b"DATA_END\nLAYER_END\n")


def make_input(shape, seed: int) -> np.ndarray:
    """N(0,1) fp32 input; CNN callers pass NCHW and convert, transformers pass [B,S,M]."""
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
