"""The five workload configurations the kernels are measured and checked on.

Shapes follow the model families runtherder supports (Llama-3.2-3B, Llama-3.1-8B, Qwen3-8B);
`int8` says whether the projections run W8A8 (per-token INT8 activations), `qk_norm` whether
q and k get Qwen3's per-head RMSNorm before RoPE.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional, Tuple


@dataclass(frozen=True)
class RopeScaling:
    factor: float = 32.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192


@dataclass(frozen=True)
class LayerConfig:
    name: str
    tokens: int            # T: token rows per call
    hidden: int            # H
    inter: int             # I
    q_heads: int
    kv_heads: int
    head_dim: int
    layers: int
    eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    int8: bool
    qk_norm: bool
    vocab: int
    seed: int
    start_pos: int = 0     # position of row 0 (decode: context depth - 1)
    max_seq: Optional[int] = None  # KV-cache slots; default tokens + start_pos

    @property
    def q_dim(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def cache_slots(self) -> int:
        return self.max_seq if self.max_seq is not None else self.tokens + self.start_pos

    def with_tokens(self, tokens: int, start_pos: Optional[int] = None) -> "LayerConfig":
        return replace(self, tokens=tokens, start_pos=self.start_pos if start_pos is None else start_pos,
                       max_seq=self.cache_slots)

    # ---- algorithmic bytes per token row (what must cross HBM at least once) ----
    def bytes_norm_quant(self) -> int:      # x, residual in; h_out bf16, codes, scale out
        return 7 * self.hidden + 4
    def bytes_norm(self) -> int:            # bf16 mode: x, residual in; h_out, y out
        return 8 * self.hidden
    def bytes_swiglu_quant(self) -> int:    # gate, up in; codes, scale out
        return 5 * self.inter + 4
    def bytes_swiglu(self) -> int:          # gate, up in; y out
        return 6 * self.inter
    def bytes_rope_kv(self) -> int:         # q,k,v + position in; q bf16, k/v fp8 + scales out
        d = self.head_dim
        return (self.q_heads + 2 * self.kv_heads) * d * 2 + 4 + self.q_heads * d * 2 + 2 * self.kv_heads * d \
            + 2 * self.kv_heads * 4
    def bytes_quant(self, k: int) -> int:   # a K-wide bf16 row in; codes, scale out
        return 3 * k + 4
    def bytes_embedding(self) -> int:       # id + row in, row out
        return 4 * self.hidden + 4

    def chain_ops(self) -> Tuple[Tuple[str, int], ...]:
        """(op name, algorithmic bytes per row) of one layer's fused-op chain, in call order."""
        if self.int8:
            return (("norm_quant", self.bytes_norm_quant()), ("rope_kv", self.bytes_rope_kv()),
                    ("quant_attn", self.bytes_quant(self.q_dim)), ("norm_quant", self.bytes_norm_quant()),
                    ("swiglu_quant", self.bytes_swiglu_quant()))
        return (("norm", self.bytes_norm()), ("rope_kv", self.bytes_rope_kv()), ("norm", self.bytes_norm()),
                ("swiglu", self.bytes_swiglu()))

    def chain_bytes_per_row(self) -> int:
        return sum(b for _, b in self.chain_ops())


_LLAMA3_SCALING = RopeScaling()

C0 = LayerConfig("c0_llama32_3b_T35", 35, 3072, 8192, 24, 8, 128, 1, 1e-5, 500000.0, _LLAMA3_SCALING, True, False,
                 128256, 0)
C1 = LayerConfig("c1_llama32_3b_prefill_T511", 511, 3072, 8192, 24, 8, 128, 28, 1e-5, 500000.0, _LLAMA3_SCALING,
                 True, False, 128256, 0)
C2 = LayerConfig("c2_llama32_3b_decode_T1_depth8196", 1, 3072, 8192, 24, 8, 128, 28, 1e-5, 500000.0,
                 _LLAMA3_SCALING, True, False, 128256, 0, start_pos=8195, max_seq=8196)
C3 = LayerConfig("c3_qwen3_8b_prefill_T8192", 8192, 4096, 12288, 32, 8, 128, 36, 1e-6, 1.0e6, None, False, True,
                 151936, 0)
C4 = LayerConfig("c4_llama31_8b_sweep_T65536", 65536, 4096, 14336, 32, 8, 128, 1, 1e-5, 500000.0, _LLAMA3_SCALING,
                 True, False, 128256, 1)

CONFIGS = {"c0": C0, "c1": C1, "c2": C2, "c3": C3, "c4": C4}
