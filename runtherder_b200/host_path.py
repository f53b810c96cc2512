"""The op chain for callers whose tensors live in HOST memory.

runtherder itself keeps activations on the device (only token ids and positions are staged from the
host, src/model/supported/llama/llama.cu:266-274), so this is not a reference interface; it exists so
the path can be driven and timed end to end from pinned host buffers.

Host format.  Rows are cut into chunks; a chunk's inputs form ONE contiguous pinned record
([x | residual | q | k | v | gate | up | ids | positions] for its rows, each field 256-byte aligned) and
its outputs another ([h_attn | q_attn_in | s_attn_in | k_cache | k_scale | v_cache | v_scale | q_mlp |
s_mlp | emb | q_rot]), so a chunk travels as one copy per direction (q is rotated in place in the input
record on the device, and is copied out from there as a second, smaller copy).  The device holds a few
record-sized slots.  Three streams — host-to-device, compute, device-to-host — each run their chunks in
order and meet through events, so neither PCIe direction ever waits for the other.  Pinned memory is
allocated with the calling thread bound to the CPUs next to the GPU (the NUMA node its PCIe root hangs
off), where the host exposes that; with eight processes copying at once, buffers on the far socket are
what limits the aggregate rate.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from . import kernels as K
from .configs import LayerConfig

# row-indexed tensors that travel per step
INPUTS_INT8 = ("x", "residual", "q", "k", "v", "gate", "up", "ids", "positions")
OUTPUTS_INT8 = ("h_attn", "q_attn_in", "s_attn_in", "k_cache", "k_scale", "v_cache", "v_scale", "q_mlp", "s_mlp", "emb")
_ALIGN = 256


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


def gpu_local_cpus(device_index: int) -> Optional[List[int]]:
    """CPUs of the NUMA node the GPU's PCIe root belongs to, from sysfs; None where that is not exposed."""
    try:
        bus = torch.cuda.get_device_properties(device_index)
        bdf = f"{bus.pci_domain_id:04x}:{bus.pci_bus_id:02x}:{bus.pci_device_id:02x}.0"
        text = open(f"/sys/bus/pci/devices/{bdf}/local_cpulist").read().strip()
    except Exception:
        return None
    cpus: List[int] = []
    for part in text.split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    allowed = os.sched_getaffinity(0)
    cpus = [c for c in cpus if c in allowed]
    return cpus or None


class _BoundTo:
    """Binds the calling thread to `cpus` for the duration of the block (first-touch places the pages of a
    pinned allocation on the node of the CPU that makes it)."""

    def __init__(self, cpus: Optional[List[int]]):
        self.cpus, self.saved = cpus, None

    def __enter__(self):
        if self.cpus:
            try:
                self.saved = os.sched_getaffinity(0)
                os.sched_setaffinity(0, self.cpus)
            except OSError:
                self.saved = None
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)


class _Record:
    """Layout of one chunk's record: name -> (byte offset, shape for n rows, dtype); fields 256-byte aligned."""

    def __init__(self, fields: List[Tuple[str, Tuple[int, ...], torch.dtype]], rows: int):
        self.rows = rows
        self.fields: Dict[str, Tuple[int, Tuple[int, ...], torch.dtype]] = {}
        off = 0
        self.payload = 0
        for name, row_shape, dtype in fields:
            shape = (rows,) + tuple(row_shape)
            nbytes = int(torch.tensor([], dtype=dtype).element_size())
            for d in shape:
                nbytes *= d
            self.fields[name] = (off, shape, dtype)
            self.payload += nbytes
            off = (off + nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        self.nbytes = off

    def views(self, block: torch.Tensor, n: Optional[int] = None) -> Dict[str, torch.Tensor]:
        """Typed views of the fields inside `block` (uint8, >= nbytes), restricted to the first n rows."""
        out = {}
        for name, (off, shape, dtype) in self.fields.items():
            count = 1
            for d in shape:
                count *= d
            esize = torch.tensor([], dtype=dtype).element_size()
            v = block[off:off + count * esize].view(dtype).view(shape)
            out[name] = v if n is None else v[:n]
        return out


class HostSweep:
    """Pinned-host in, pinned-host out execution of `sweep_step` over `rows` token rows."""

    def __init__(self, cfg: LayerConfig, rows: int, weights: Dict[str, torch.Tensor], chunk_rows: int = 4096,
                 n_slots: int = 3, device="cuda"):
        self.cfg, self.rows, self.weights = cfg, rows, weights
        self.chunk = min(chunk_rows, rows)
        self.dev = torch.device(device)
        self.n_chunks = (rows + self.chunk - 1) // self.chunk
        self.n_slots = max(2, min(n_slots, self.n_chunks + 1))
        H, I, D = cfg.hidden, cfg.inter, cfg.head_dim
        bf, i8, f32, u8, i32 = torch.bfloat16, torch.int8, torch.float32, torch.uint8, torch.int32
        self.rec_in = _Record([("x", (H,), bf), ("residual", (H,), bf), ("q", (cfg.q_heads, D), bf),
                               ("k", (cfg.kv_heads, D), bf), ("v", (cfg.kv_heads, D), bf), ("gate", (I,), bf),
                               ("up", (I,), bf), ("ids", (), i32), ("positions", (), i32)], self.chunk)
        self.rec_out = _Record([("h_attn", (H,), bf), ("q_attn_in", (H,), i8), ("s_attn_in", (), f32),
                                ("k_cache", (cfg.kv_heads, D), u8), ("k_scale", (cfg.kv_heads,), f32),
                                ("v_cache", (cfg.kv_heads, D), u8), ("v_scale", (cfg.kv_heads,), f32),
                                ("q_mlp", (I,), i8), ("s_mlp", (), f32), ("emb", (H,), bf)], self.chunk)
        self.q_off, q_shape, _ = self.rec_in.fields["q"]
        self.q_row_bytes = cfg.q_heads * D * 2
        self.cpus = gpu_local_cpus(self.dev.index or 0)
        with torch.cuda.device(self.dev):
            self.h2d, self.compute, self.d2h = (torch.cuda.Stream(device=self.dev) for _ in range(3))
            self.slot_in = [torch.empty(self.rec_in.nbytes, dtype=u8, device=self.dev) for _ in range(self.n_slots)]
            self.slot_out = [torch.empty(self.rec_out.nbytes, dtype=u8, device=self.dev) for _ in range(self.n_slots)]
            self.at_pos = torch.zeros(1, dtype=i32, device=self.dev)
            ev = lambda: [torch.cuda.Event() for _ in range(self.n_slots)]
            self.ev_in, self.ev_done, self.ev_out = ev(), ev(), ev()

    # ---- host buffers --------------------------------------------------------------------------------
    def _pinned(self, nbytes: int) -> torch.Tensor:
        with _BoundTo(self.cpus):
            t = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
            t[::4096] = 0          # touch every page from a CPU next to the GPU
        return t

    def alloc_host_inputs(self, device_inputs: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        """One pinned record per chunk, filled from row-indexed device tensors (set-up, not timed)."""
        blocks = []
        stage = self.slot_in[0]
        for c in range(self.n_chunks):
            b = c * self.chunk
            n = min(self.chunk, self.rows - b)
            views = self.rec_in.views(stage, n)
            for name in INPUTS_INT8:
                views[name].copy_(device_inputs[name][b:b + n])
            host = self._pinned(self.rec_in.nbytes)
            host.copy_(stage)
            blocks.append(host)
        torch.cuda.synchronize(self.dev)
        return blocks

    def alloc_host_outputs(self) -> List[torch.Tensor]:
        """One pinned record per chunk: the output fields followed by the rotated q rows."""
        return [self._pinned(self.rec_out.nbytes + self.chunk * self.q_row_bytes) for _ in range(self.n_chunks)]

    def unpack_outputs(self, host_out: List[torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Row-indexed host tensors assembled from the output records (for checks; copies)."""
        parts: Dict[str, List[torch.Tensor]] = {name: [] for name in OUTPUTS_INT8 + ("q_rot",)}
        for c, block in enumerate(host_out):
            n = min(self.chunk, self.rows - c * self.chunk)
            for name, v in self.rec_out.views(block, n).items():
                parts[name].append(v.clone())
            q = block[self.rec_out.nbytes:self.rec_out.nbytes + n * self.q_row_bytes].view(torch.bfloat16)
            parts["q_rot"].append(q.view(n, self.cfg.q_heads, self.cfg.head_dim).clone())
        return {name: torch.cat(v, dim=0) for name, v in parts.items()}

    def bytes_per_step(self) -> Tuple[int, int]:
        """(host-to-device, device-to-host) payload bytes of one step, padding excluded."""
        per_row_in = self.rec_in.payload // self.chunk
        per_row_out = self.rec_out.payload // self.chunk + self.q_row_bytes
        return per_row_in * self.rows, per_row_out * self.rows

    # ---- one step ------------------------------------------------------------------------------------
    def run(self, host_in: List[torch.Tensor], host_out: List[torch.Tensor]) -> int:
        """Enqueues everything and returns the number of kernel launches; the caller synchronises
        (torch.cuda.synchronize or wait on the current stream) before reading host_out."""
        launches = 0
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.h2d, self.compute, self.d2h):
            s.wait_stream(cur)
        for c in range(self.n_chunks):
            n = min(self.chunk, self.rows - c * self.chunk)
            slot = c % self.n_slots
            reuse = c >= self.n_slots
            with torch.cuda.stream(self.h2d):
                if reuse:                      # the slot's input record was read by compute and by the q copy-out
                    self.h2d.wait_event(self.ev_out[slot])
                self.slot_in[slot].copy_(host_in[c], non_blocking=True)
                self.ev_in[slot].record(self.h2d)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(self.ev_in[slot])
                if reuse:                      # the slot's output record must have left
                    self.compute.wait_event(self.ev_out[slot])
                i = self.rec_in.views(self.slot_in[slot], n)
                i.update(self.weights)
                o = self.rec_out.views(self.slot_out[slot], n)
                o["at_pos"] = self.at_pos
                launches += sweep_step(self.cfg, i, o)
                self.ev_done[slot].record(self.compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.ev_done[slot])
                host_out[c][:self.rec_out.nbytes].copy_(self.slot_out[slot], non_blocking=True)
                qb = n * self.q_row_bytes
                host_out[c][self.rec_out.nbytes:self.rec_out.nbytes + qb].copy_(
                    self.slot_in[slot][self.q_off:self.q_off + qb], non_blocking=True)
                self.ev_out[slot].record(self.d2h)
        for s in (self.h2d, self.compute, self.d2h):
            cur.wait_stream(s)
        return launches
