"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: bf16 activations ~N(0,1) with 0.5 % of the hidden channels scaled x20, norm
gains ~U(0.5,1.5), token ids ~U[0,vocab), embedding table ~N(0,0.02).

Values come from the library's counter-based device generators (rh_synth_*), so element i of a
tensor depends only on (seed, tensor id, i): a row shard generated on another GPU, or a slice
regenerated on the host, is bit-identical to the same rows of the full tensor.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ._lib import call
from .configs import LayerConfig
from .kernels import _stream
from .rope_tables import inv_freq_for

from .synth_spec import (OUTLIER_FRACTION, OUTLIER_SCALE, T_ATTN, T_G_ATTN, T_G_FFN, T_GATE, T_IDS, T_K, T_KNORM,  # noqa: F401
                         T_Q, T_QNORM, T_RES, T_TABLE, T_UP, T_V, T_X, outlier_channel_scale)


def normal_bf16(count: int, seed: int, tensor_id: int, start: int = 0, std: float = 1.0,
                chan_scale: Optional[torch.Tensor] = None, ncols: int = 1, device="cuda", out=None) -> torch.Tensor:
    out = torch.empty(count, dtype=torch.bfloat16, device=device) if out is None else out
    call("rh_synth_normal_bf16", out.data_ptr(), count, seed, tensor_id, start, std,
         None if chan_scale is None else chan_scale.data_ptr(), ncols, _stream(None))
    return out


def uniform_bf16(count: int, seed: int, tensor_id: int, lo: float, hi: float, start: int = 0, device="cuda"):
    out = torch.empty(count, dtype=torch.bfloat16, device=device)
    call("rh_synth_uniform_bf16", out.data_ptr(), count, seed, tensor_id, start, lo, hi, _stream(None))
    return out


def ids_i32(count: int, seed: int, tensor_id: int, modulus: int, start: int = 0, device="cuda"):
    out = torch.empty(count, dtype=torch.int32, device=device)
    call("rh_synth_ids_i32", out.data_ptr(), count, seed, tensor_id, start, modulus, _stream(None))
    return out


def make_inputs(cfg: LayerConfig, rows: Optional[int] = None, row_offset: int = 0, device="cuda",
                with_table: bool = True) -> Dict[str, torch.Tensor]:
    """Inputs of one layer's op chain for global token rows [row_offset, row_offset+rows).

    Row-indexed tensors are slices of the full T-row tensors of `cfg`; weights (gains, inv_freq,
    embedding table) are the replicated full tensors.  positions are global: start_pos + row.
    """
    T = cfg.tokens if rows is None else rows
    H, I, D = cfg.hidden, cfg.inter, cfg.head_dim
    s = cfg.seed
    dev = torch.device(device)
    with torch.cuda.device(dev):
        def act(tid, width, outliers=False):
            cs = None
            if outliers:
                cs = torch.from_numpy(outlier_channel_scale(width, s, tid)).to(dev)
            return normal_bf16(T * width, s, tid, start=row_offset * width, chan_scale=cs, ncols=width,
                               device=dev).view(T, width)

        d = {
            "x": act(T_X, H, True), "residual": act(T_RES, H, True),
            "g_attn": uniform_bf16(H, s, T_G_ATTN, 0.5, 1.5, device=dev),
            "g_ffn": uniform_bf16(H, s, T_G_FFN, 0.5, 1.5, device=dev),
            "q": act(T_Q, cfg.q_dim).view(T, cfg.q_heads, D),
            "k": act(T_K, cfg.kv_dim).view(T, cfg.kv_heads, D),
            "v": act(T_V, cfg.kv_dim).view(T, cfg.kv_heads, D),
            "gate": act(T_GATE, I), "up": act(T_UP, I),
            "attn": act(T_ATTN, cfg.q_dim),
            "ids": ids_i32(T, s, T_IDS, cfg.vocab, start=row_offset, device=dev),
            "positions": torch.arange(cfg.start_pos + row_offset, cfg.start_pos + row_offset + T, dtype=torch.int32,
                                      device=dev),
            "inv_freq": torch.from_numpy(inv_freq_for(cfg)).to(dev),
        }
        if cfg.qk_norm:
            d["q_norm"] = uniform_bf16(D, s, T_QNORM, 0.5, 1.5, device=dev)
            d["k_norm"] = uniform_bf16(D, s, T_KNORM, 0.5, 1.5, device=dev)
        if with_table:
            d["table"] = normal_bf16(cfg.vocab * H, s, T_TABLE, std=0.02, device=dev).view(cfg.vocab, H)
    return d
