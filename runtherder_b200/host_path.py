"""The op chain for callers whose tensors live in HOST memory.

runtherder itself keeps activations on the device (only token ids and positions are staged from the
host, src/model/supported/llama/llama.cu:266-274), so this is not a reference interface; it exists so
the path can be driven and timed end to end from pinned host buffers.  Rows are cut into chunks; each
chunk's inputs are copied to the device, run through the fused kernels and copied back, with chunks
rotating over a few streams so the two PCIe directions and the kernels overlap.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from . import kernels as K
from .configs import LayerConfig

# row-indexed tensors that travel per step
INPUTS_INT8 = ("x", "residual", "q", "k", "v", "gate", "up", "ids", "positions")
OUTPUTS_INT8 = ("h_attn", "q_attn_in", "s_attn_in", "q_rot", "k_cache", "k_scale", "v_cache", "v_scale", "q_mlp",
                "s_mlp", "emb")


def sweep_step(cfg: LayerConfig, i: Dict[str, torch.Tensor], o: Dict[str, torch.Tensor], stream=None) -> int:
    """The four ops of the throughput sweep, one launch each: embedding gather, residual add + RMSNorm +
    INT8, RoPE + FP8 KV append, SwiGLU + INT8.  q is rotated in place.  Returns the launch count."""
    T, H = i["x"].shape
    K.embedding_lookup_bf16_forward(o["emb"], i["table"], i["ids"], T, H, stream)
    K.rmsnorm_add_quant_int8(o["q_attn_in"], o["s_attn_in"], o["h_attn"], None, i["x"], i["residual"], i["g_attn"],
                             T, H, cfg.eps, stream)
    K.rope_kv_fp8(i["q"], None, i["k"], i["v"], i.get("q_norm"), i.get("k_norm"), cfg.eps, i["positions"],
                  i["inv_freq"], o["k_cache"], o["k_scale"], o["v_cache"], o["v_scale"], o["at_pos"], T, cfg.q_heads,
                  cfg.kv_heads, cfg.head_dim, stream)
    K.swiglu_quant_int8(o["q_mlp"], o["s_mlp"], None, i["gate"], i["up"], T, cfg.inter, stream)
    return 4


class HostSweep:
    """Pinned-host in, pinned-host out execution of `sweep_step` over `rows` token rows."""

    def __init__(self, cfg: LayerConfig, rows: int, weights: Dict[str, torch.Tensor], chunk_rows: int = 4096,
                 n_streams: int = 3, device="cuda"):
        from .layer_ops import alloc_outputs
        self.cfg, self.rows, self.weights = cfg, rows, weights
        self.chunk = min(chunk_rows, rows)
        self.dev = torch.device(device)
        self.streams = [torch.cuda.Stream(device=self.dev) for _ in range(n_streams)]
        H, I, D = cfg.hidden, cfg.inter, cfg.head_dim
        shapes = {"x": (H,), "residual": (H,), "q": (cfg.q_heads, D), "k": (cfg.kv_heads, D), "v": (cfg.kv_heads, D),
                  "gate": (I,), "up": (I,)}
        self.stage_in: List[Dict[str, torch.Tensor]] = []
        self.stage_out: List[Dict[str, torch.Tensor]] = []
        for _ in range(n_streams):
            d = {k: torch.empty((self.chunk,) + s, dtype=torch.bfloat16, device=self.dev) for k, s in shapes.items()}
            d["ids"] = torch.empty(self.chunk, dtype=torch.int32, device=self.dev)
            d["positions"] = torch.empty(self.chunk, dtype=torch.int32, device=self.dev)
            d.update(weights)
            self.stage_in.append(d)
            o = alloc_outputs(cfg, self.chunk, device=self.dev, slots=self.chunk)
            self.stage_out.append(o)

    def alloc_host_outputs(self) -> Dict[str, torch.Tensor]:
        o = self.stage_out[0]
        host = {}
        for name in OUTPUTS_INT8:
            src = self.stage_in[0]["q"] if name == "q_rot" else o[name]
            host[name] = torch.empty((self.rows,) + tuple(src.shape[1:]), dtype=src.dtype).pin_memory()
        return host

    def bytes_per_step(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor]):
        h2d = sum(host_in[k].numel() * host_in[k].element_size() for k in INPUTS_INT8)
        d2h = sum(v.numel() * v.element_size() for v in host_out.values())
        return h2d, d2h

    def run(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor]) -> int:
        """One step.  Enqueues everything and returns the number of kernel launches; the caller
        synchronises (torch.cuda.synchronize or the streams) before reading host_out."""
        launches = 0
        cur = torch.cuda.current_stream(self.dev)
        for s in self.streams:
            s.wait_stream(cur)
        for c, begin in enumerate(range(0, self.rows, self.chunk)):
            n = min(self.chunk, self.rows - begin)
            slot = c % len(self.streams)
            st, din, dout = self.streams[slot], self.stage_in[slot], self.stage_out[slot]
            with torch.cuda.stream(st):
                i = dict(din)
                for k in INPUTS_INT8:
                    i[k] = din[k][:n]
                    i[k].copy_(host_in[k][begin:begin + n], non_blocking=True)
                o = {k: (v[:n] if v.dim() and v.shape[0] == self.chunk and k != "at_pos" else v) for k, v in dout.items()}
                launches += sweep_step(self.cfg, i, o)
                for name in OUTPUTS_INT8:
                    src = i["q"] if name == "q_rot" else o[name]
                    host_out[name][begin:begin + n].copy_(src, non_blocking=True)
        for s in self.streams:
            cur.wait_stream(s)
        return launches
