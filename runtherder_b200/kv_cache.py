"""FP8 E4M3 KV cache with per-(token, kv_head) scales — the slab layout and append rule of
runtherder's engine::KVCache (include/runtherder/engine/kv_cache.h:18-22, 62-89).

K and V slabs are [num_layers, max_seq_len, num_kv_heads, head_dim] E4M3 bytes; the scale slabs
[num_layers, max_seq_len, num_kv_heads] fp32.  The write position is a device-resident int32 so a
captured CUDA graph picks up a new position on every replay; like the reference, the device does
not check it against max_seq_len — `append` callers own that bound (`check_bound` helps).
"""
from __future__ import annotations

import torch

from . import kernels as K
from ._lib import RhError


class KVCache:
    def __init__(self, num_layers: int, max_seq_len: int, num_kv_heads: int, head_dim: int, device="cuda"):
        for name, v in (("num_layers", num_layers), ("max_seq_len", max_seq_len), ("num_kv_heads", num_kv_heads),
                        ("head_dim", head_dim)):
            if v < 1:
                raise RhError("KVCache", 1, f"KVCache {name} must be >= 1")
        self.num_layers, self.max_seq_len = num_layers, max_seq_len
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        shape = (num_layers, max_seq_len, num_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=torch.uint8, device=device)
        self.v = torch.zeros(shape, dtype=torch.uint8, device=device)
        self.k_scale = torch.zeros(shape[:3], dtype=torch.float32, device=device)
        self.v_scale = torch.zeros(shape[:3], dtype=torch.float32, device=device)

    def _layer(self, layer: int):
        if not 0 <= layer < self.num_layers:
            raise RhError("KVCache", 1, "KVCache layer out of range")
        return self.k[layer], self.v[layer], self.k_scale[layer], self.v_scale[layer]

    def check_bound(self, start_pos: int, n_new: int) -> None:
        """The host-side bound the reference checks in LlamaModel::stage (llama.cu:263-264)."""
        if start_pos < 0 or start_pos + n_new > self.max_seq_len:
            raise RhError("KVCache", 1, f"positions {start_pos}..{start_pos + n_new} exceed max_seq_len "
                                        f"{self.max_seq_len}")

    def append(self, layer: int, k, v, n_new: int, at_pos, stream=None) -> None:
        """Quantise n_new bf16 keys and values into `layer` at row *at_pos (kv_cache.h:62-78):
        two quantize_kv_fp8 calls, exactly as the reference issues them."""
        if n_new < 1:
            raise RhError("KVCache", 1, "KVCache append n_new must be >= 1")
        if at_pos is None:
            raise RhError("KVCache", 1, "KVCache append at_pos must not be null")
        kc, vc, ks, vs = self._layer(layer)
        rows = n_new * self.num_kv_heads
        K.quantize_kv_fp8(kc, ks, k, at_pos, self.num_kv_heads, rows, self.head_dim, stream)
        K.quantize_kv_fp8(vc, vs, v, at_pos, self.num_kv_heads, rows, self.head_dim, stream)

    def rope_append(self, layer: int, q, k, v, positions, inv_freq, n_new: int, at_pos, num_q_heads: int,
                    q_norm=None, k_norm=None, eps: float = 1e-6, k_out=None, stream=None) -> None:
        """Fused path: [QK-norm +] RoPE on q (in place) and k, then the append of rotated k and of v."""
        kc, vc, ks, vs = self._layer(layer)
        K.rope_kv_fp8(q, k_out, k, v, q_norm, k_norm, eps, positions, inv_freq, kc, ks, vc, vs, at_pos, n_new,
                      num_q_heads, self.num_kv_heads, self.head_dim, stream)

    def view(self, layer: int):
        """(k, v, k_scale, v_scale) of one layer — what attention kernels consume (kv_cache.h:80-89)."""
        return self._layer(layer)
