"""Python mirror of runtherder's kernel API (namespace runtherder::kernels).

Function names, argument order and argument meaning follow the reference headers
include/runtherder/kernels/{rmsnorm,quantization,rope,activation,embedding}.cuh; the
fused entry points at the bottom are additions.  Tensors are torch CUDA tensors (or raw
device addresses as int); every call only enqueues work on `stream` (default: torch's
current stream) and raises RhError where the reference would print and exit.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ._lib import RhError, call

TensorOrPtr = Union[torch.Tensor, int, None]

__all__ = [
    "RhError", "rmsnorm_bf16_forward", "rmsnorm_add_bf16_forward", "quantize_per_token_int8",
    "dequantize_w8a8", "quantize_kv_fp8", "dequantize_kv_fp8", "swiglu_bf16_forward", "rope_bf16",
    "embedding_lookup_bf16_forward", "qkv_bias_add_bf16_forward", "stage_positions", "decode_advance",
    "flash_split_scratch_floats", "flash_decode_split_bf16", "flash_prefill_bf16", "tune", "bias_rope_kv_fp8", "rmsnorm_add_quant_int8", "swiglu_quant_int8", "rope_kv_fp8",
    "rmsnorm_add_last_row", "init",
]


def _ptr(t: TensorOrPtr, dtype: Optional[torch.dtype] = None, numel: Optional[int] = None, name: str = "tensor"):
    """Device address of `t`, after the host-side checks a C++ caller gets from the type system."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not t.is_cuda:
        raise RhError(name, 1, f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RhError(name, 1, f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RhError(name, 1, f"{name} must have dtype {dtype}, got {t.dtype}")
    if numel is not None and t.numel() < numel:
        raise RhError(name, 1, f"{name} holds {t.numel()} elements, {numel} needed")
    return t.data_ptr()


def _stream(stream) -> Optional[int]:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream or None
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream or None
    return int(stream) or None


_BF, _I8, _I32, _F32, _U8 = torch.bfloat16, torch.int8, torch.int32, torch.float32, torch.uint8
_FP8 = (torch.uint8, torch.float8_e4m3fn)


def _fp8_ptr(t, numel, name):
    if isinstance(t, torch.Tensor) and t.dtype not in _FP8:
        raise RhError(name, 1, f"{name} must be uint8 or float8_e4m3fn, got {t.dtype}")
    return _ptr(t, None, numel, name)


def tune(key: str, value: int) -> None:
    """Set a process-wide tuning knob of the library (`rh_tune`); value <= 0 restores the default."""
    call("rh_tune", key.encode(), int(value))


def rmsnorm_bf16_forward(y, x, g, num_tokens: int, hidden_dim: int, eps: float, stream=None) -> None:
    """y = (x / rms(x)) * g; y may alias x.  (rmsnorm.cuh:15-22)"""
    n = num_tokens * hidden_dim
    call("rh_rmsnorm_bf16", _ptr(y, _BF, n, "y"), _ptr(x, _BF, n, "x"), _ptr(g, _BF, hidden_dim, "g"),
         num_tokens, hidden_dim, eps, _stream(stream))


def rmsnorm_add_bf16_forward(y, h_out, x, residual, g, num_tokens: int, hidden_dim: int, eps: float,
                             stream=None) -> None:
    """h_out = x + residual, y = rmsnorm(h_out) * g; h_out may alias residual.  (rmsnorm.cuh:36-45)"""
    n = num_tokens * hidden_dim
    call("rh_rmsnorm_add_bf16", _ptr(y, _BF, n, "y"), _ptr(h_out, _BF, n, "h_out"), _ptr(x, _BF, n, "x"),
         _ptr(residual, _BF, n, "residual"), _ptr(g, _BF, hidden_dim, "g"), num_tokens, hidden_dim, eps,
         _stream(stream))


def rmsnorm_add_last_row(y_last, x, residual, g, num_tokens: int, hidden_dim: int, eps: float, stream=None) -> None:
    """y_last[hidden_dim] = row num_tokens-1 of rmsnorm(x + residual) * g: the final norm when only the last
    token feeds lm_head (llama3.cu:254-263 normalises every row and slices)."""
    n = num_tokens * hidden_dim
    call("rh_rmsnorm_add_last_row_bf16", _ptr(y_last, _BF, hidden_dim, "y_last"), _ptr(x, _BF, n, "x"),
         _ptr(residual, _BF, n, "residual"), _ptr(g, _BF, hidden_dim, "g"), num_tokens, hidden_dim, eps, _stream(stream))


def device_error() -> int:
    """rh_device_error: the sticky per-device word a bounded wait records into when it gives up
    ((source line << 8) | 1; 0 = no kernel has given up so far).  Synchronises the device."""
    import ctypes
    word = ctypes.c_int(-1)
    call("rh_device_error", ctypes.byref(word))
    return int(word.value)


def init(device: int = 0) -> None:
    """rh_init: makes every kernel of the library resident and set up on `device`, so that even the first
    call of an entry point may be recorded into a CUDA graph."""
    call("rh_init", int(device))


def quantize_per_token_int8(q, x_scale, x, num_tokens: int, dim: int, stream=None) -> None:
    """q = round(x / x_scale), x_scale = row amax / 127.  (quantization.cuh:17-22)"""
    n = num_tokens * dim
    call("rh_quantize_per_token_int8", _ptr(q, _I8, n, "q"), _ptr(x_scale, _F32, num_tokens, "x_scale"),
         _ptr(x, _BF, n, "x"), num_tokens, dim, _stream(stream))


def dequantize_w8a8(y, acc, x_scale, w_scale, m: int, n: int, stream=None) -> None:
    """y = acc * x_scale[row] * w_scale[col].  (quantization.cuh:31-37)"""
    call("rh_dequantize_w8a8", _ptr(y, _BF, m * n, "y"), _ptr(acc, _I32, m * n, "acc"),
         _ptr(x_scale, _F32, m, "x_scale"), _ptr(w_scale, _BF, n, "w_scale"), m, n, _stream(stream))


def quantize_kv_fp8(q, scale, x, at_pos, rows_per_pos: int, num_rows: int, head_dim: int, stream=None) -> None:
    """E4M3 rows with scale = amax/448, written from row at_pos*rows_per_pos on; at_pos is a
    device-resident int32.  (quantization.cuh:50-57)"""
    call("rh_quantize_kv_fp8", _fp8_ptr(q, None, "q"), _ptr(scale, _F32, None, "scale"),
         _ptr(x, _BF, num_rows * head_dim, "x"), _ptr(at_pos, _I32, 1, "at_pos"), rows_per_pos, num_rows,
         head_dim, _stream(stream))


def dequantize_kv_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """float(q) * scale, the read side of the KV cache (quantization.cuh:63-66).  q: [..., D] E4M3
    bytes, scale: [...] fp32.  Convenience for tests and cache consumers written in torch."""
    return q.view(torch.float8_e4m3fn).to(torch.float32) * scale.unsqueeze(-1)


def swiglu_bf16_forward(y, gate, up, n: int, stream=None) -> None:
    """y[i] = silu(gate[i]) * up[i]; y may alias gate or up.  (activation.cuh:16-21)"""
    call("rh_swiglu_bf16", _ptr(y, _BF, n, "y"), _ptr(gate, _BF, n, "gate"), _ptr(up, _BF, n, "up"), n,
         _stream(stream))


def rope_bf16(q, k, positions, inv_freq, seq_len: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
              stream=None) -> None:
    """In-place RoPE on q [T,Hq,D] and k [T,Hkv,D]; token t rotates by positions[t].  (rope.cuh:16-25)"""
    call("rh_rope_bf16", _ptr(q, _BF, seq_len * num_q_heads * head_dim, "q"),
         _ptr(k, _BF, seq_len * num_kv_heads * head_dim, "k"), _ptr(positions, _I32, seq_len, "positions"),
         _ptr(inv_freq, _F32, head_dim // 2, "inv_freq"), seq_len, num_q_heads, num_kv_heads, head_dim,
         _stream(stream))


def embedding_lookup_bf16_forward(out, embedding_table, token_ids, num_tokens: int, hidden_dim: int,
                                  stream=None) -> None:
    """out[i] = embedding_table[token_ids[i]].  (embedding.cuh:14-20)"""
    call("rh_embedding_lookup_bf16", _ptr(out, _BF, num_tokens * hidden_dim, "out"),
         _ptr(embedding_table, _BF, hidden_dim, "embedding_table"), _ptr(token_ids, _I32, num_tokens, "token_ids"),
         num_tokens, hidden_dim, _stream(stream))


def qkv_bias_add_bf16_forward(q, k, v, q_bias, k_bias, v_bias, n: int, q_dim: int, kv_dim: int, stream=None) -> None:
    """q[r] += q_bias, k[r] += k_bias, v[r] += v_bias for every row, in place.  (bias.cuh:20-30)"""
    call("rh_qkv_bias_add_bf16", _ptr(q, _BF, n * q_dim, "q"), _ptr(k, _BF, n * kv_dim, "k"), _ptr(v, _BF, n * kv_dim, "v"),
         _ptr(q_bias, _BF, q_dim, "q_bias"), _ptr(k_bias, _BF, kv_dim, "k_bias"), _ptr(v_bias, _BF, kv_dim, "v_bias"),
         n, q_dim, kv_dim, _stream(stream))


def stage_positions(positions, decode_pos, start_pos: int, n: int, stream=None) -> None:
    """positions[:n] = start_pos + arange(n), decode_pos[0] = start_pos, on the device (llama.cu:266-274)."""
    call("rh_stage_positions", _ptr(positions, _I32, n, "positions"), _ptr(decode_pos, _I32, 1, "decode_pos"), start_pos, n,
         _stream(stream))


def decode_advance(token_slot, position, decode_pos, next_token, step: int = 1, stream=None) -> None:
    """token_slot[0] = next_token[0]; position[0] += step; decode_pos[0] += step — graph-capturable step update."""
    call("rh_decode_advance", _ptr(token_slot, _I32, 1, "token_slot"), _ptr(position, _I32, 1, "position"),
         _ptr(decode_pos, _I32, 1, "decode_pos"), _ptr(next_token, _I32, 1, "next_token"), step, _stream(stream))


def flash_split_scratch_floats(num_q_heads: int, head_dim: int, max_splits: int) -> int:
    """Floats of scratch a split decode needs (flash_decode.cuh:11-25)."""
    from ._lib import lib
    return int(lib.rh_flash_split_scratch_floats(num_q_heads, head_dim, max_splits))


def flash_decode_split_bf16(out, q, k, v, k_scale, v_scale, partial, num_splits: int, cache_len, num_q_heads: int,
                            num_kv_heads: int, head_dim: int, scale: float, stream=None) -> None:
    """One query token attends keys 0..*cache_len of the FP8 cache; cache_len is a device-resident int32,
    partial caller-owned fp32 scratch of flash_split_scratch_floats(...) floats.  (flash_decode.cuh:27-62)"""
    need = flash_split_scratch_floats(num_q_heads, head_dim, num_splits)
    call("rh_flash_decode_split_bf16", _ptr(out, _BF, num_q_heads * head_dim, "out"),
         _ptr(q, _BF, num_q_heads * head_dim, "q"), _fp8_ptr(k, None, "k"), _fp8_ptr(v, None, "v"),
         _ptr(k_scale, _F32, None, "k_scale"), _ptr(v_scale, _F32, None, "v_scale"),
         _ptr(partial, _F32, need, "partial"), num_splits, _ptr(cache_len, _I32, 1, "cache_len"), num_q_heads,
         num_kv_heads, head_dim, float(scale), _stream(stream))


def flash_prefill_bf16(out, q, k, v, k_scale, v_scale, n_new: int, cache_len, num_q_heads: int, num_kv_heads: int,
                       head_dim: int, scale: float, stream=None) -> None:
    """n_new query tokens attend causally over the FP8 cache (token t sees keys 0..*cache_len + t); cache_len is
    a device-resident int32.  head_dim 128.  (flash_prefill.cuh:27-40)"""
    call("rh_flash_prefill_bf16", _ptr(out, _BF, n_new * num_q_heads * head_dim, "out"),
         _ptr(q, _BF, n_new * num_q_heads * head_dim, "q"), _fp8_ptr(k, None, "k"), _fp8_ptr(v, None, "v"),
         _ptr(k_scale, _F32, None, "k_scale"), _ptr(v_scale, _F32, None, "v_scale"), n_new,
         _ptr(cache_len, _I32, 1, "cache_len"), num_q_heads, num_kv_heads, head_dim, float(scale), _stream(stream))


# ---- fused entry points ---------------------------------------------------------------------

def rmsnorm_add_quant_int8(q, x_scale, h_out, y, x, residual, g, num_tokens: int, hidden_dim: int, eps: float,
                           stream=None) -> None:
    """[residual add +] RMSNorm + per-token INT8 in one pass; equals rmsnorm(_add)_bf16_forward followed
    by quantize_per_token_int8 of the stored result.  residual=None: plain norm; y=None: no bf16 store."""
    n = num_tokens * hidden_dim
    call("rh_rmsnorm_add_quant_int8", _ptr(q, _I8, n, "q"), _ptr(x_scale, _F32, num_tokens, "x_scale"),
         _ptr(h_out, _BF, n, "h_out"), _ptr(y, _BF, n, "y"), _ptr(x, _BF, n, "x"),
         _ptr(residual, _BF, n, "residual"), _ptr(g, _BF, hidden_dim, "g"), num_tokens, hidden_dim, eps,
         _stream(stream))


def swiglu_quant_int8(q, x_scale, y, gate, up, num_tokens: int, inter_dim: int, stream=None) -> None:
    """SwiGLU + per-token INT8 of the bf16-rounded product; y=None skips the bf16 store."""
    n = num_tokens * inter_dim
    call("rh_swiglu_quant_int8", _ptr(q, _I8, n, "q"), _ptr(x_scale, _F32, num_tokens, "x_scale"),
         _ptr(y, _BF, n, "y"), _ptr(gate, _BF, n, "gate"), _ptr(up, _BF, n, "up"), num_tokens, inter_dim,
         _stream(stream))


def rope_kv_fp8(q, k_out, k_in, v_in, q_norm, k_norm, eps: float, positions, inv_freq, k_cache, k_scale,
                v_cache, v_scale, at_pos, seq_len: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                stream=None) -> None:
    """[per-head RMSNorm of q,k +] RoPE + FP8 KV-cache append of rotated k and of v at slot *at_pos."""
    nq, nk = seq_len * num_q_heads * head_dim, seq_len * num_kv_heads * head_dim
    call("rh_rope_kv_fp8", _ptr(q, _BF, nq, "q"), _ptr(k_out, _BF, nk, "k_out"), _ptr(k_in, _BF, nk, "k_in"),
         _ptr(v_in, _BF, nk, "v_in"), _ptr(q_norm, _BF, head_dim, "q_norm"), _ptr(k_norm, _BF, head_dim, "k_norm"),
         eps, _ptr(positions, _I32, seq_len, "positions"), _ptr(inv_freq, _F32, head_dim // 2, "inv_freq"),
         _fp8_ptr(k_cache, None, "k_cache"), _ptr(k_scale, _F32, None, "k_scale"),
         _fp8_ptr(v_cache, None, "v_cache"), _ptr(v_scale, _F32, None, "v_scale"), _ptr(at_pos, _I32, 1, "at_pos"),
         seq_len, num_q_heads, num_kv_heads, head_dim, _stream(stream))


def bias_rope_kv_fp8(q, k_out, k_in, v_in, q_bias, k_bias, v_bias, positions, inv_freq, k_cache, k_scale, v_cache,
                     v_scale, at_pos, seq_len: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                     stream=None) -> None:
    """Qwen2: projection biases + RoPE + FP8 KV-cache append in one launch; equals qkv_bias_add_bf16_forward
    followed by rope_kv_fp8 (v_in is left unmodified)."""
    nq, nk = seq_len * num_q_heads * head_dim, seq_len * num_kv_heads * head_dim
    call("rh_bias_rope_kv_fp8", _ptr(q, _BF, nq, "q"), _ptr(k_out, _BF, nk, "k_out"), _ptr(k_in, _BF, nk, "k_in"),
         _ptr(v_in, _BF, nk, "v_in"), _ptr(q_bias, _BF, num_q_heads * head_dim, "q_bias"),
         _ptr(k_bias, _BF, num_kv_heads * head_dim, "k_bias"), _ptr(v_bias, _BF, num_kv_heads * head_dim, "v_bias"),
         _ptr(positions, _I32, seq_len, "positions"), _ptr(inv_freq, _F32, head_dim // 2, "inv_freq"),
         _fp8_ptr(k_cache, None, "k_cache"), _ptr(k_scale, _F32, None, "k_scale"),
         _fp8_ptr(v_cache, None, "v_cache"), _ptr(v_scale, _F32, None, "v_scale"), _ptr(at_pos, _I32, 1, "at_pos"),
         seq_len, num_q_heads, num_kv_heads, head_dim, _stream(stream))
