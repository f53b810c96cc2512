"""One decoder layer's row-wise op chain, as runtherder's layer composition issues it
(src/model/supported/llama/llama3.cu:208-252, qwen3.cu:169-222), in two forms:

* `fused_layer_step`  — the fused entry points: 5 launches per W8A8 layer (norm+quant, rope+kv,
  quant of the attention output, norm+quant, swiglu+quant), 4 per bf16 layer.
* `reference_sequence` — the reference's own call sequence through an object exposing the
  reference's function names (this package's `kernels` module, or the reference's CUDA kernels
  in the tests): 13 launches per W8A8 layer, because quantize_per_token_int8 lives inside every
  linear_w8a8 (src/kernels/matmul.cu:138) and re-quantises the same rows for q/k/v and gate/up.

The GEMMs and attention between these ops are not part of the path; their outputs (q, k, v, the
attention output, gate, up, the MLP output x) are inputs here.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import kernels as K
from .configs import LayerConfig


def alloc_outputs(cfg: LayerConfig, rows: int, device="cuda", slots: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Output buffers of one layer for `rows` token rows; the KV slabs hold `slots` positions."""
    dev = torch.device(device)
    slots = rows if slots is None else slots
    H, I = cfg.hidden, cfg.inter
    o = {
        "h_attn": torch.empty(rows, H, dtype=torch.bfloat16, device=dev),
        "h_ffn": torch.empty(rows, H, dtype=torch.bfloat16, device=dev),
        "k_cache": torch.zeros(slots, cfg.kv_heads, cfg.head_dim, dtype=torch.uint8, device=dev),
        "v_cache": torch.zeros(slots, cfg.kv_heads, cfg.head_dim, dtype=torch.uint8, device=dev),
        "k_scale": torch.zeros(slots, cfg.kv_heads, dtype=torch.float32, device=dev),
        "v_scale": torch.zeros(slots, cfg.kv_heads, dtype=torch.float32, device=dev),
        "at_pos": torch.zeros(1, dtype=torch.int32, device=dev),
        "emb": torch.empty(rows, H, dtype=torch.bfloat16, device=dev),
    }
    if cfg.int8:
        o.update({
            "q_attn_in": torch.empty(rows, H, dtype=torch.int8, device=dev),
            "s_attn_in": torch.empty(rows, dtype=torch.float32, device=dev),
            "q_attn_out": torch.empty(rows, cfg.q_dim, dtype=torch.int8, device=dev),
            "s_attn_out": torch.empty(rows, dtype=torch.float32, device=dev),
            "q_ffn_in": torch.empty(rows, H, dtype=torch.int8, device=dev),
            "s_ffn_in": torch.empty(rows, dtype=torch.float32, device=dev),
            "q_mlp": torch.empty(rows, I, dtype=torch.int8, device=dev),
            "s_mlp": torch.empty(rows, dtype=torch.float32, device=dev),
        })
    else:
        o.update({
            "normed": torch.empty(rows, H, dtype=torch.bfloat16, device=dev),
            "ffn_normed": torch.empty(rows, H, dtype=torch.bfloat16, device=dev),
            "mlp_act": torch.empty(rows, I, dtype=torch.bfloat16, device=dev),
        })
    return o


ATTENTION_SPLITS = 32   # what the reference's AdaptiveAttention passes (src/attention/adaptive.cu:13)


def attention_step(api, cfg: LayerConfig, i: Dict[str, torch.Tensor], o: Dict[str, torch.Tensor], partial: torch.Tensor,
                   stream=None) -> int:
    """The attention between the KV append and the quantisation of its output, as AdaptiveAttention dispatches
    it (src/attention/adaptive.cu:24-41): split-KV flash decode for one token, flash prefill otherwise.  Reads
    the rotated q and the layer's cache, with *at_pos as the number of keys cached before these tokens; writes
    i["attn"].  `api` offers the reference's function names.  Returns the number of kernels launched."""
    import math
    T = i["x"].shape[0]
    scale = 1.0 / math.sqrt(cfg.head_dim)
    if T == 1:
        api.flash_decode_split_bf16(i["attn"], i["q"], o["k_cache"], o["v_cache"], o["k_scale"], o["v_scale"], partial,
                                    ATTENTION_SPLITS, o["at_pos"], cfg.q_heads, cfg.kv_heads, cfg.head_dim, scale, stream)
        return 2
    api.flash_prefill_bf16(i["attn"], i["q"], o["k_cache"], o["v_cache"], o["k_scale"], o["v_scale"], T, o["at_pos"],
                           cfg.q_heads, cfg.kv_heads, cfg.head_dim, scale, stream)
    return 1


def fused_layer_step(cfg: LayerConfig, i: Dict[str, torch.Tensor], o: Dict[str, torch.Tensor], stream=None,
                     with_embedding: bool = False, attention_partial: Optional[torch.Tensor] = None) -> int:
    """Enqueue one layer's fused chain; returns the number of kernels launched.  With `attention_partial`
    (fp32 scratch of flash_split_scratch_floats(Hq, D, ATTENTION_SPLITS) floats) the attention over the FP8
    cache runs between the KV append and the quantisation of its output.

    Reads i[x, residual, q, k, v, attn, gate, up, ...]; q is rotated in place; h_attn / h_ffn receive
    the updated residual stream (the reference passes h_out == residual; separate buffers here keep the
    inputs intact so a step can be repeated and checked)."""
    T, H = i["x"].shape
    n = 0
    if with_embedding:
        K.embedding_lookup_bf16_forward(o["emb"], i["table"], i["ids"], T, H, stream)
        n += 1
    if cfg.int8:
        K.rmsnorm_add_quant_int8(o["q_attn_in"], o["s_attn_in"], o["h_attn"], None, i["x"], i["residual"],
                                 i["g_attn"], T, H, cfg.eps, stream)
    else:
        K.rmsnorm_add_bf16_forward(o["normed"], o["h_attn"], i["x"], i["residual"], i["g_attn"], T, H, cfg.eps,
                                   stream)
    K.rope_kv_fp8(i["q"], None, i["k"], i["v"], i.get("q_norm"), i.get("k_norm"), cfg.eps, i["positions"],
                  i["inv_freq"], o["k_cache"], o["k_scale"], o["v_cache"], o["v_scale"], o["at_pos"], T,
                  cfg.q_heads, cfg.kv_heads, cfg.head_dim, stream)
    n += 2
    if attention_partial is not None:
        n += attention_step(K, cfg, i, o, attention_partial, stream)
    if cfg.int8:
        K.quantize_per_token_int8(o["q_attn_out"], o["s_attn_out"], i["attn"], T, cfg.q_dim, stream)
        K.rmsnorm_add_quant_int8(o["q_ffn_in"], o["s_ffn_in"], o["h_ffn"], None, i["x"], o["h_attn"], i["g_ffn"], T, H,
                                 cfg.eps, stream)
        K.swiglu_quant_int8(o["q_mlp"], o["s_mlp"], None, i["gate"], i["up"], T, cfg.inter, stream)
        n += 3
    else:
        K.rmsnorm_add_bf16_forward(o["ffn_normed"], o["h_ffn"], i["x"], o["h_attn"], i["g_ffn"], T, H, cfg.eps,
                                   stream)
        K.swiglu_bf16_forward(o["mlp_act"], i["gate"], i["up"], T * cfg.inter, stream)
        n += 2
    return n


def reference_sequence(api, cfg: LayerConfig, i: Dict[str, torch.Tensor], o: Dict[str, torch.Tensor],
                       scratch: Dict[str, torch.Tensor], stream=None, dedup_quant: bool = False,
                       attention_partial: Optional[torch.Tensor] = None) -> int:
    """The same layer through the reference's own call sequence.  `api` offers the reference's function
    names.  scratch: bf16 `normed`, `ffn_normed`, `act` [T,I] and (int8) `q8` [T,max K], `s8` [T].
    With dedup_quant the repeated quantisation of the same rows (x3 for q/k/v, x2 for gate/up) is
    issued once.  Outputs land in the same `o` buffers as the fused step, q/k are rotated in place."""
    T, H = i["x"].shape
    I, D = cfg.inter, cfg.head_dim
    n = 0

    def quant(dst_q, dst_s, src, k, times):
        nonlocal n
        for _ in range(1 if dedup_quant else times):
            api.quantize_per_token_int8(dst_q, dst_s, src, T, k, stream)
            n += 1

    # bf16 models keep the normalised rows (they feed the bf16 GEMMs); W8A8 models only need them as the
    # quantiser's input
    normed = scratch["normed"] if cfg.int8 else o["normed"]
    ffn_normed = scratch["ffn_normed"] if cfg.int8 else o["ffn_normed"]
    act = scratch["act"] if cfg.int8 else o["mlp_act"]
    api.rmsnorm_add_bf16_forward(normed, o["h_attn"], i["x"], i["residual"], i["g_attn"], T, H, cfg.eps, stream)
    n += 1
    if cfg.int8:
        quant(o["q_attn_in"], o["s_attn_in"], normed, H, 3)
    if cfg.qk_norm:
        api.rmsnorm_bf16_forward(i["q"], i["q"], i["q_norm"], T * cfg.q_heads, D, cfg.eps, stream)
        api.rmsnorm_bf16_forward(i["k"], i["k"], i["k_norm"], T * cfg.kv_heads, D, cfg.eps, stream)
        n += 2
    api.rope_bf16(i["q"], i["k"], i["positions"], i["inv_freq"], T, cfg.q_heads, cfg.kv_heads, D, stream)
    api.quantize_kv_fp8(o["k_cache"], o["k_scale"], i["k"], o["at_pos"], cfg.kv_heads, T * cfg.kv_heads, D, stream)
    api.quantize_kv_fp8(o["v_cache"], o["v_scale"], i["v"], o["at_pos"], cfg.kv_heads, T * cfg.kv_heads, D, stream)
    n += 3
    if attention_partial is not None:
        n += attention_step(api, cfg, i, o, attention_partial, stream)
    if cfg.int8:
        quant(o["q_attn_out"], o["s_attn_out"], i["attn"], cfg.q_dim, 1)
    api.rmsnorm_add_bf16_forward(ffn_normed, o["h_ffn"], i["x"], o["h_attn"], i["g_ffn"], T, H, cfg.eps, stream)
    n += 1
    if cfg.int8:
        quant(o["q_ffn_in"], o["s_ffn_in"], ffn_normed, H, 2)
    api.swiglu_bf16_forward(act, i["gate"], i["up"], T * I, stream)
    n += 1
    if cfg.int8:
        quant(o["q_mlp"], o["s_mlp"], act, I, 1)
    return n
