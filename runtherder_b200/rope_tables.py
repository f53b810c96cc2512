"""Host-side RoPE frequency tables (load-time work in runtherder: LlamaModel builds the
table once and uploads it; the kernels only ever see the table).

rope_inv_freq_plain  <- src/model/supported/llama/llama.cu:128-143
rope_inv_freq_llama3 <- src/model/supported/llama/llama3.cu:26-60
Both are computed by the native library (double precision, then narrowed to float).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import call
from .configs import LayerConfig, RopeScaling


def rope_inv_freq_plain(head_dim: int, theta_base: float) -> np.ndarray:
    out = np.empty(max(head_dim // 2, 0), dtype=np.float32)
    call("rh_rope_inv_freq_plain", out.ctypes.data_as(C.c_void_p), head_dim, theta_base)
    return out


def rope_inv_freq_llama3(head_dim: int, theta_base: float, scaling: RopeScaling) -> np.ndarray:
    out = np.empty(max(head_dim // 2, 0), dtype=np.float32)
    call("rh_rope_inv_freq_llama3", out.ctypes.data_as(C.c_void_p), head_dim, theta_base, scaling.factor,
         scaling.low_freq_factor, scaling.high_freq_factor, scaling.original_max_position_embeddings)
    return out


def inv_freq_for(cfg: LayerConfig) -> np.ndarray:
    """The table LlamaModel::arrange would upload for this config (llama3.cu:106-110)."""
    if cfg.rope_scaling is not None:
        return rope_inv_freq_llama3(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
    return rope_inv_freq_plain(cfg.head_dim, cfg.rope_theta)
