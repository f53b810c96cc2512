"""Which synthetic tensor is which, and which hidden channels are outliers: the pure-numpy part of the
synthetic inputs, kept free of the native library so that a host-only consumer (the CPU reference arm of
the benchmark) can regenerate any slice without loading CUDA code."""
from __future__ import annotations

import math

import numpy as np

# tensor ids (the generator's stream selector)
T_X, T_RES, T_G_ATTN, T_G_FFN, T_Q, T_K, T_V, T_GATE, T_UP, T_ATTN, T_TABLE, T_IDS, T_QNORM, T_KNORM = range(1, 15)

OUTLIER_FRACTION = 0.005
OUTLIER_SCALE = 20.0


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def outlier_channel_scale(ncols: int, seed: int, tensor_id: int) -> np.ndarray:
    """fp32 [ncols]: 20.0 on ceil(0.5 %) channels picked once per tensor from the seed, 1.0 elsewhere."""
    n_out = math.ceil(OUTLIER_FRACTION * ncols)
    with np.errstate(over="ignore"):
        key = np.uint64((seed * 0x9E3779B97F4A7C15 + tensor_id * 0xD1B54A32D192ED03 + 0x1234567) % (1 << 64))
        h = _mix64(np.arange(ncols, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15) + key)
    scale = np.ones(ncols, dtype=np.float32)
    scale[np.argsort(h, kind="stable")[:n_out]] = OUTLIER_SCALE
    return scale
