#!/usr/bin/env python
"""Benchmark of the fused row-wise layer ops on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (default N=1)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU implementation

Workload (config.workload): the Llama-3.1-8B-shaped throughput sweep — T=65536 token rows, hidden 4096,
32 Q / 8 KV heads x 128, intermediate 14336, vocab 128256, seed 1.  A step is one pass of its four ops
over the batch, one launch each: embedding gather, residual add + RMSNorm + INT8 quantisation, llama3
RoPE + FP8 KV append, SwiGLU + INT8 quantisation.  With N GPUs the rows are split into N contiguous
blocks (strong scaling, no collective on the data path).

value  = algorithmic HBM bytes of a step / device time of the step, whole job (GB/s), inputs resident.
         The K-step region (no event, no host work between launches) is timed `--repeats` times, each
         bracketed by a barrier and a synchronise; ms_per_step is the median region, the spread is reported.
ops    = per-kernel times from separate passes with an event after every launch: one straight after the
         warm-up (kernels alone, in a burst: what `roofline` uses) and one after the timed regions (sustained).
e2e    = the same bytes / wall time of a step driven from pinned HOST buffers (H2D + kernels + D2H).
verify = (N > 1) rows around every shard boundary, gathered over NCCL from the GPUs that own them and
         compared bit for bit with the same rows computed on rank 0 alone; outside the timed region.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fused-layer-op HBM GB/s"
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0


def dram_traffic_per_row(kernel: str, rows: int):
    """dram__bytes_read.sum + dram__bytes_write.sum per token row of a step kernel, from the ncu captures listed
    in profiles/dram_traffic.json (one entry per (kernel, rows) actually captured).  Rows are independent units,
    so a launch's traffic is the per-row figure of the nearest captured row count times its rows; None when the
    kernel was never captured."""
    f = ROOT / "profiles" / "dram_traffic.json"
    try:
        entries = [e for e in json.loads(f.read_text())["captures"] if e["kernel"] == kernel]
    except Exception:
        return None
    if not entries:
        return None
    best = min(entries, key=lambda e: abs(e["rows"] - rows))
    return (best["dram_bytes_read"] + best["dram_bytes_write"]) / best["rows"]


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--config", default="c4")
    p.add_argument("--rows", type=int, default=0, help="override the row count (smaller captures)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--no-refcuda", action="store_true")
    p.add_argument("--no-secondary", action="store_true", help="skip the attention timings appended to the sweep line")
    p.add_argument("--no-verify", action="store_true", help="N > 1: skip the cross-GPU check of the shard boundaries")
    p.add_argument("--repeats", type=int, default=5, help="how many times the K-step region is timed (median reported)")
    p.add_argument("--cpu-seconds", type=float, default=15.0)
    p.add_argument("--graph", choices=["auto", "on", "off"], default="auto",
                   help="layer-chain configs: replay the forward from a CUDA graph (auto: on for the decode config)")
    p.add_argument("--attention", action="store_true",
                   help="time the attention over the FP8 cache instead of the row-wise chain (secondary line; not the "
                        "headline metric): the split-KV flash decode for --config c2 (or any config with --depth), "
                        "the causal prefill for configs with more than one token (c1, c3)")
    p.add_argument("--with-attention", action="store_true",
                   help="layer-chain configs: run the attention over the FP8 cache inside every layer (flash decode for "
                        "the decode config, flash prefill otherwise), between the KV append and the quantisation of its output")
    p.add_argument("--depth", type=int, default=0, help="--attention: override the context depth (keys attended)")
    p.add_argument("--splits", type=int, default=32, help="--attention: split count (the reference uses 32)")
    p.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                   help="set a library tuning knob (rh_tune) before measuring, e.g. no_pdl=1; repeatable")
    return p.parse_args()


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def note_device_error(line):
    """Reads the library's sticky device error word into the line; a kernel whose bounded wait gave up has
    produced no valid result, so a non-zero word ends the run instead of reporting a number."""
    from runtherder_b200 import kernels as Kn
    word = Kn.device_error()
    line["device_error"] = word
    if word != 0:
        raise SystemExit(f"bench: a kernel gave up a bounded wait (device error word {word:#x}, source line {word >> 8})")


def sweep_config(cfg, world, rows_per_gpu):
    """The `config` object of the throughput-sweep line; both arms print the same one."""
    ops, per_row = step_bytes_per_row(cfg)
    return {"workload": cfg.name, "token_rows": cfg.tokens, "rows_per_gpu": rows_per_gpu, "hidden": cfg.hidden,
            "inter": cfg.inter, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
            "vocab": cfg.vocab, "seed": cfg.seed, "ops_per_step": [n for n, _ in ops],
            "algorithmic_bytes_per_row": per_row, "parallelism": f"rows/{world}",
            "l2": "every op streams more than the 126 MB L2 per launch (inputs larger than L2)"}


def step_bytes_per_row(cfg):
    ops = [("embedding", cfg.bytes_embedding()), ("norm_quant", cfg.bytes_norm_quant()),
           ("rope_kv", cfg.bytes_rope_kv()), ("swiglu_quant", cfg.bytes_swiglu_quant())]
    return ops, sum(b for _, b in ops)


# ------------------------------------------------------------------------------------------------
# clocks: sampled through NVML (read-only) while the timed region runs
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.period = period_s

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's host implementation (its test helpers, compiled unmodified) where it
# has one, the oracle port for the pieces it lacks (INT8 quantisation, gather); rows over all cores.
# ------------------------------------------------------------------------------------------------
def cpu_rows_per_second(cfg, total_rows: int, threads: int):
    """Runs the four ops of a step on `total_rows` synthetic rows on the host; returns (seconds, kind)."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    from oracle_lib import Oracle, load_ref_host, ptr
    from runtherder_b200 import synth_spec as synth      # numpy only: this arm never loads the CUDA library

    orc = Oracle()
    ref = load_ref_host()
    H, I, D, Hq, Hkv = cfg.hidden, cfg.inter, cfg.head_dim, cfg.q_heads, cfg.kv_heads
    s = cfg.seed
    g = orc.synth_uniform(H, s, synth.T_G_ATTN, 0.5, 1.5)
    table_rows = 4096                                     # a window of the table: the gather cost is per row
    table = orc.synth_normal(table_rows * H, s, synth.T_TABLE, 0, 0.02).reshape(table_rows, H)
    cs = synth.outlier_channel_scale(H, s, synth.T_X)

    def work(block):
        b, e = block
        n = e - b
        x = orc.synth_normal(n * H, s, synth.T_X, b * H, 1.0, cs, H).reshape(n, H)
        r = orc.synth_normal(n * H, s, synth.T_RES, b * H, 1.0, cs, H).reshape(n, H)
        q = orc.synth_normal(n * Hq * D, s, synth.T_Q, b * Hq * D).reshape(n, Hq, D)
        k = orc.synth_normal(n * Hkv * D, s, synth.T_K, b * Hkv * D).reshape(n, Hkv, D)
        v = orc.synth_normal(n * Hkv * D, s, synth.T_V, b * Hkv * D).reshape(n * Hkv, D)
        gate = orc.synth_normal(n * I, s, synth.T_GATE, b * I).reshape(n, I)
        up = orc.synth_normal(n * I, s, synth.T_UP, b * I).reshape(n, I)
        ids = (orc.synth_ids(n, s, synth.T_IDS, cfg.vocab, b) % table_rows).astype(np.int32)
        t0 = time.perf_counter()
        orc.embedding(table, ids)
        if ref is not None:
            y, h = np.empty_like(x), np.empty_like(x)
            ref.refhost_rmsnorm_add(ptr(y), ptr(h), ptr(x), ptr(r), ptr(g), n, H, cfg.eps)
        else:
            y, h = orc.rmsnorm_add(x, r, g, cfg.eps)
        orc.quant_int8(y)
        if ref is not None:   # the reference's host RoPE takes theta and a start position (plain table)
            ref.refhost_rope(ptr(q), cfg.start_pos + b, n, Hq, D, cfg.rope_theta)
            ref.refhost_rope(ptr(k), cfg.start_pos + b, n, Hkv, D, cfg.rope_theta)
            kq, ks = np.empty(n * Hkv * D, np.uint8), np.empty(n * Hkv, np.float32)
            ref.refhost_quantize_kv(ptr(kq), ptr(ks), ptr(k), n * Hkv, D)
            ref.refhost_quantize_kv(ptr(kq), ptr(ks), ptr(v), n * Hkv, D)
            act = np.empty_like(gate)
            ref.refhost_swiglu(ptr(act), ptr(gate), ptr(up), n * I)
        else:
            pos = np.arange(cfg.start_pos + b, cfg.start_pos + e, dtype=np.int32)
            rs = cfg.rope_scaling
            inv = (orc.inv_freq_plain(D, cfg.rope_theta) if rs is None else
                   orc.inv_freq_llama3(D, cfg.rope_theta, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
                                       rs.original_max_position_embeddings))
            orc.rope_table(q, pos, inv)
            k = orc.rope_table(k, pos, inv)
            orc.quant_kv(k.reshape(n * Hkv, D))
            orc.quant_kv(v)
            act = orc.swiglu(gate, up)
        orc.quant_int8(act)
        return time.perf_counter() - t0

    per = max(1, total_rows // threads)
    blocks = [(b, min(total_rows, b + per)) for b in range(0, total_rows, per)]
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as pool:
        busy = list(pool.map(work, blocks))
    wall = time.perf_counter() - t0
    # input generation is not part of the measured work: scale the wall time by the busy share
    gen_overhead = max(0.0, wall - max(busy))
    return max(busy), ("reference" if ref is not None else "port"), gen_overhead


def cpu_baseline(cfg, seconds: float):
    threads = os.cpu_count() or 1
    probe_rows = 4 * threads
    t, kind, _ = cpu_rows_per_second(cfg, probe_rows, threads)
    rate = probe_rows / max(t, 1e-9)
    rows = int(min(max(rate * seconds, 8 * threads), 65536))
    rows -= rows % threads
    t, kind, _ = cpu_rows_per_second(cfg, rows, threads)
    _, per_row = step_bytes_per_row(cfg)
    one_rows = max(16, min(512, int(rate / threads * 3.0)))        # ~3 s of the scalar code as the reference has it
    t1, _, _ = cpu_rows_per_second(cfg, one_rows, 1)
    return {"value": rows * per_row / t / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "rows_per_s": rows / t,
            "single_thread": {"value": one_rows * per_row / t1 / 1e9, "unit": "GB/s", "rows_per_s": one_rows / t1,
                              "sample": f"{one_rows} rows on one thread"},
            "sample": f"{rows} of {cfg.tokens} token rows of the same four ops, row-parallel over {threads} host "
                      f"threads; {'reference test helpers (double precision) for norm, RoPE, FP8 KV, SwiGLU; ' if kind == 'reference' else ''}"
                      f"oracle port for INT8 quantisation and the gather (the reference has no host code for them); "
                      f"{'RoPE through the plain-theta table its host helper builds (no llama3 rescaling), ' if kind == 'reference' else ''}"
                      f"gather from a 4096-row window of the table"}


def run_reference_arm(args, cfg):
    """The reference's own CPU implementation of the path, timed in K bounded steps on this host."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    _, per_row = step_bytes_per_row(cfg)
    budget = 90.0
    probe_rows = 4 * threads
    t, kind, _ = cpu_rows_per_second(cfg, probe_rows, threads)
    rate = probe_rows / max(t, 1e-9)
    rows = int(min(max(rate * budget / (args.steps + args.warmup), 2 * threads), 16384))
    rows -= rows % threads
    for _ in range(args.warmup):
        cpu_rows_per_second(cfg, rows, threads)
    total = 0.0
    for _ in range(args.steps):
        t, kind, _ = cpu_rows_per_second(cfg, rows, threads)
        total += t
    ms = total / args.steps * 1e3
    value = rows * per_row / (total / args.steps) / 1e9
    sample = (f"each step = {rows} of {cfg.tokens} token rows through the four ops on {threads} host threads "
              f"(reference test helpers where the reference has host code, oracle port for INT8 quantisation and gather; "
              f"RoPE through the plain-theta table the reference's host helper builds, gather from a 4096-row window of the table)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64",
            "io_dtypes": "bf16 in; int8 / fp8-e4m3 / bf16 out (the reference's host helpers compute in double)",
            "data": "synthetic", "token_rows_per_s": rows / (total / args.steps),
            "config": sweep_config(cfg, args.gpus, -(-cfg.tokens // max(args.gpus, 1))), "sample_rows_per_step": rows,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    from runtherder_b200.configs import CONFIGS
    cfg = CONFIGS[args.config]
    if args.rows:
        cfg = cfg.with_tokens(args.rows)
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    import torch
    import torch.distributed as dist
    from runtherder_b200 import host_path, kernels, layer_ops, synth
    from runtherder_b200.sharding import shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    for item in args.tune:
        key, _, value = item.partition("=")
        kernels.tune(key, int(value))
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep stdout for the one JSON line
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.attention:
        if world != 1:
            raise SystemExit("--attention is a single-GPU measurement (one query token does not shard)")
        if cfg.tokens > 1 and not args.depth:
            run_prefill_attention(args, cfg, dev)
        else:
            run_decode_attention(args, cfg, dev)
        return
    if args.config != "c4":
        run_layer_chain(args, cfg, world, rank, dev, barrier, max_over_ranks)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    T = cfg.tokens
    b, e = shard_bounds(T, world, rank)
    rows = e - b
    ops, per_row = step_bytes_per_row(cfg)
    ins = synth.make_inputs(cfg, rows=rows, row_offset=b, device=dev)
    outs = layer_ops.alloc_outputs(cfg, rows, device=dev, slots=rows)
    torch.cuda.synchronize()

    def step():
        return host_path.sweep_step(cfg, ins, outs)

    for _ in range(max(args.warmup, 3)):
        step()
    K = args.steps
    # The timed loop calls the C ABI directly with pre-resolved device pointers (the Python mirror in
    # runtherder_b200.kernels adds ~10 us of argument checking per call, which matters once a GPU's share
    # of a step shrinks to ~200 us at 8 GPUs).
    from runtherder_b200 import _lib
    L = _lib.lib
    sp = torch.cuda.current_stream().cuda_stream or None
    H = cfg.hidden
    P = lambda t: t.data_ptr()
    calls = [
        (L.rh_embedding_lookup_bf16, (P(outs["emb"]), P(ins["table"]), P(ins["ids"]), rows, H, sp)),
        (L.rh_rmsnorm_add_quant_int8, (P(outs["q_attn_in"]), P(outs["s_attn_in"]), P(outs["h_attn"]), None, P(ins["x"]),
                                       P(ins["residual"]), P(ins["g_attn"]), rows, H, cfg.eps, sp)),
        (L.rh_rope_kv_fp8, (P(ins["q"]), None, P(ins["k"]), P(ins["v"]), None, None, cfg.eps, P(ins["positions"]),
                            P(ins["inv_freq"]), P(outs["k_cache"]), P(outs["k_scale"]), P(outs["v_cache"]),
                            P(outs["v_scale"]), P(outs["at_pos"]), rows, cfg.q_heads, cfg.kv_heads, cfg.head_dim, sp)),
        (L.rh_swiglu_quant_int8, (P(outs["q_mlp"]), P(outs["s_mlp"]), None, P(ins["gate"]), P(ins["up"]), rows, cfg.inter, sp)),
    ]
    status = 0

    def per_kernel_pass(steps):
        """An event after every launch (this serialises the kernels, so it is never part of a timed region):
        each kernel's median duration over `steps` steps, max over ranks."""
        nonlocal status
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
        barrier()
        for s_ in range(steps):
            e_ = ev[s_]
            e_[0].record()
            for j, (fn, fargs) in enumerate(calls):
                status |= fn(*fargs)
                e_[j + 1].record()
        torch.cuda.synchronize()
        barrier()
        ms = [statistics.median(ev[s_][j].elapsed_time(ev[s_][j + 1]) for s_ in range(steps)) for j in range(4)]
        return [max_over_ranks(m) for m in ms]

    # ---- per-kernel pass, kernels timed alone straight after the warm-up (the condition the copy peak they
    # are held against was measured in: a short burst) ----
    op_ms = per_kernel_pass(min(K, 20))

    # ---- timed regions: K steps each, nothing but the four launches per step between the two events, so the
    # kernels keep their programmatic-dependent-launch overlap; a barrier and a synchronise on both sides ----
    launches = 0
    region_ms = []
    t_enqueue = 0.0
    with ClockSampler(local_rank) as clocks:
        for _ in range(max(1, args.repeats)):
            first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            t0 = time.perf_counter()
            first.record()
            for _s in range(K):
                for fn, fargs in calls:
                    status |= fn(*fargs)
            last.record()
            t_enqueue += time.perf_counter() - t0
            torch.cuda.synchronize()
            barrier()
            region_ms.append(max_over_ranks(first.elapsed_time(last)))
            launches += 4 * K
    per_step = sorted(ms / K for ms in region_ms)
    ms_per_step = statistics.median(per_step)
    spread = {"repeats": len(per_step), "ms_per_step_all": [round(ms / K, 4) for ms in region_ms],
              "min": round(per_step[0], 4), "max": round(per_step[-1], 4),
              "iqr": round(per_step[(3 * len(per_step)) // 4] - per_step[len(per_step) // 4], 4)}

    # ---- the same per-kernel pass again, now on a GPU that has been streaming for the whole run: where the
    # board reaches its power cap the SM clock is lower and a kernel that needs instruction issue shows it ----
    op_ms_sustained = per_kernel_pass(K)
    if status != 0:
        raise SystemExit("a kernel call failed: " + L.rh_last_error_string().decode())

    peak, peak_kind = measured_peak()
    total_bytes = T * per_row
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    op_table = {}
    for (name, bpr), ms, ms_hot in zip(ops, op_ms, op_ms_sustained):
        # per-GPU figures: this rank's rows / its kernel time (max over ranks)
        gbs, gbs_hot = rows * bpr / (ms * 1e-3) / 1e9, rows * bpr / (ms_hot * 1e-3) / 1e9
        op_table[name] = {"ms": round(ms, 4), "gbs_per_gpu": round(gbs, 1), "frac_of_" + peak_kind: round(gbs / peak, 4),
                          "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4), "bytes_per_row": bpr,
                          "sustained": {"ms": round(ms_hot, 4), "frac_of_" + peak_kind: round(gbs_hot / peak, 4)}}
    dom = max(range(4), key=lambda j: op_ms[j])
    dom_name, dom_bpr = ops[dom]
    achieved = rows * dom_bpr / (op_ms[dom] * 1e-3) / 1e9
    achieved_hot = rows * dom_bpr / (op_ms_sustained[dom] * 1e-3) / 1e9
    traffic = dram_traffic_per_row(dom_name, rows) if args.config == "c4" else None
    traffic = None if traffic is None else int(traffic * rows)
    roofline = {"bound": "hbm", "kernel": dom_name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}", "traffic": traffic,
                "algorithmic_bytes_per_launch": rows * dom_bpr,
                "sustained": {"achieved": round(achieved_hot, 1), "frac": round(achieved_hot / peak, 4),
                              "what": "the same kernel timed the same way after the timed regions, on a GPU that has been "
                                      "streaming for the whole run (SM clock and throttle reasons: see clocks)"},
                "timing": "median launch duration of a per-kernel pass (an event after every launch) run straight after the "
                          "warm-up, separate from the timed regions: the kernel alone, in a short burst, as the copy peak was measured"}

    line = {"metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "io_dtypes": "bf16 in; int8 codes, fp8-e4m3 cache bytes, fp32 scales, bf16 out",
            "data": "synthetic", "token_rows_per_s": round(T / (ms_per_step * 1e-3), 1),
            "frac_of_hbm_peak": {peak_kind: round(value / (peak * world), 4),
                                 "nominal_8TBs": round(value / (NOMINAL_HBM_GBS * world), 4)},
            "config": sweep_config(cfg, world, rows), "timed_regions": spread,
            "ops": op_table, "roofline": roofline, "gpu_launches": launches, "clocks": clocks.summary(),
            "host_enqueue_us_per_step": round(t_enqueue / (K * max(1, args.repeats)) * 1e6, 1)}

    # ---- N > 1: the shards' bytes against the same rows computed on rank 0 alone ----
    if world > 1 and not args.no_verify:
        line["verify"] = verify_shards(cfg, ins, outs, b, rows, world, rank, dev, calls)

    # ---- the reference's own CUDA kernels on the same buffers (rank 0, N=1) ----
    if world == 1 and not args.no_refcuda:
        try:
            line["ref_cuda"] = time_reference_cuda(cfg, ins, outs, rows, per_row, max(3, min(K, 20)))
        except Exception as exc:  # library absent: report, do not fail the bench
            line["ref_cuda"] = {"unavailable": str(exc)[:200]}

    # ---- end to end from pinned host buffers ----
    if not args.no_e2e:
        line["e2e"] = time_end_to_end(cfg, ins, rows, total_bytes, world, barrier, max_over_ranks,
                                      steps=max(3, min(K, 8)), dev=dev)

    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(cfg, args.cpu_seconds)
    # ---- secondary: the attention kernels over the FP8 cache (the consumers of this path's bytes), N = 1 ----
    if world == 1 and not args.no_secondary and args.config == "c4" and not args.rows:
        del ins, outs
        torch.cuda.empty_cache()
        line["secondary"] = secondary_attention(args, dev)
    note_device_error(line)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def secondary_attention(args, dev):
    """Short timings of the two attention kernels on their own configurations, appended to the sweep line so
    that one bench run records them: causal prefill on the Qwen3-8B prefill shape (TFLOP/s) and the split-KV
    decode at depth 8196 inside a 28-layer CUDA graph (us per call).  Not part of the headline metric."""
    import copy
    from runtherder_b200.configs import CONFIGS
    sub = copy.copy(args)
    sub.steps, sub.warmup, sub.no_refcuda, sub.no_cpu, sub.depth = 10, 3, True, True, 0
    out = {}
    for key, cfg_name, fn in (("prefill_c3", "c3", run_prefill_attention), ("decode_c2", "c2", run_decode_attention)):
        try:
            ln = fn(sub, CONFIGS[cfg_name], dev, emit=False)
            out[key] = {k: ln[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "config", "roofline", "gpu_launches")
                        if k in ln}
            if "us_per_call" in ln:
                out[key]["us_per_call"] = ln["us_per_call"]
        except Exception as exc:
            out[key] = {"unavailable": str(exc)[:200]}
    return out


def verify_shards(cfg, ins, outs, begin, rows, world, rank, dev, calls):
    """After an N-GPU run: for a window of rows around every shard boundary (and the first and last rows),
    gather each output's rows over NCCL from the ranks that own them and compare them, bit for bit, with
    the same rows computed by rank 0 alone from freshly generated inputs.  The rotated q is produced in
    place (and therefore re-rotated by every step), so its comparison uses a fresh single pass on every
    rank; all other outputs are the timed buffers themselves."""
    import torch
    from runtherder_b200 import host_path, layer_ops, synth
    from runtherder_b200.sharding import boundary_windows, gather_window
    T = cfg.tokens
    names = ["emb", "h_attn", "q_attn_in", "s_attn_in", "k_cache", "k_scale", "v_cache", "v_scale", "q_mlp", "s_mlp"]
    weights = {k: ins[k] for k in ("g_attn", "inv_freq", "table")}
    ok, checked_rows, bad = True, 0, []
    # a fresh single pass over this rank's rows for the in-place output
    q_fresh = synth.make_inputs(cfg, rows=rows, row_offset=begin, device=dev, with_table=False)
    q_fresh.update(weights)
    scratch = layer_ops.alloc_outputs(cfg, rows, device=dev, slots=rows)
    host_path.sweep_step(cfg, q_fresh, scratch)
    torch.cuda.synchronize()
    local = {n: outs[n] for n in names}
    local["q_rot"] = q_fresh["q"]
    for lo, hi in boundary_windows(T, world, half_width=64):
        gathered = {n: gather_window(t, T, lo, hi) for n, t in local.items()}
        if rank == 0:
            one = synth.make_inputs(cfg, rows=hi - lo, row_offset=lo, device=dev, with_table=False)
            one.update(weights)
            ref = layer_ops.alloc_outputs(cfg, hi - lo, device=dev, slots=hi - lo)
            host_path.sweep_step(cfg, one, ref)
            torch.cuda.synchronize()
            ref["q_rot"] = one["q"]
            for n, g in gathered.items():
                same = torch.equal(g.contiguous().view(torch.uint8), ref[n].contiguous().view(torch.uint8))
                if not same:
                    ok = False
                    bad.append(f"{n}[{lo}:{hi}]")
            checked_rows += hi - lo
    return {"ok": ok, "rows": checked_rows, "outputs": list(local.keys()), "mismatches": bad[:8],
            "how": "rows around every shard boundary gathered over NCCL from their owners vs the same rows computed on rank 0 alone, bitwise"}


def run_layer_chain(args, cfg, world, rank, dev, barrier, max_over_ranks):
    """Configs c0-c3: a step is one forward's worth of the per-layer op chain — the embedding gather, then
    `layers` x (fused norm[+INT8], RoPE[+QK-norm]+FP8 KV append, [INT8 of the attention output,] fused
    norm[+INT8], SwiGLU[+INT8]) — on rotating buffer sets (distinct memory per layer up to ~2 GB, never
    fewer than two sets) so a layer does not find its inputs in L2 from the previous one.  Timed eagerly
    and, for the decode config, as one CUDA graph.  The reference's own CUDA kernels run the same forward
    through the reference's call sequence (13 launches per W8A8 layer) for comparison."""
    import torch
    from runtherder_b200 import layer_ops, synth
    from runtherder_b200.sharding import shard_bounds

    T, L = cfg.tokens, cfg.layers
    b, e = shard_bounds(T, world, rank)
    rows = e - b
    if rows == 0:
        raise SystemExit(f"{cfg.name}: fewer rows than ranks")
    per_row = cfg.chain_bytes_per_row()
    layer_bytes = per_row * rows * 2.2            # inputs + outputs + scratch, roughly
    n_sets = int(min(L, max(2, 2e9 // max(layer_bytes, 1))))
    sub = cfg.with_tokens(rows, start_pos=cfg.start_pos)
    ins = [synth.make_inputs(sub, rows=rows, row_offset=b + i * 7, device=dev, with_table=(i == 0)) for i in range(n_sets)]
    slots = cfg.cache_slots
    outs = [layer_ops.alloc_outputs(cfg, rows, device=dev, slots=slots) for _ in range(n_sets)]
    for o in outs:
        o["at_pos"].fill_(cfg.start_pos + b)
    for i in ins:
        i["positions"] = torch.arange(cfg.start_pos + b, cfg.start_pos + e, dtype=torch.int32, device=dev)
    partial = None
    if args.with_attention:
        if world != 1:
            raise SystemExit("--with-attention is a single-GPU measurement (attention does not shard by rows)")
        from runtherder_b200 import kernels as Kn
        partial = torch.empty(Kn.flash_split_scratch_floats(cfg.q_heads, cfg.head_dim, layer_ops.ATTENTION_SPLITS),
                              dtype=torch.float32, device=dev)
        if cfg.start_pos > 0:      # decode: give every layer's cache a seeded history to attend
            gen = torch.Generator(device=dev).manual_seed(cfg.seed + 79)
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            for o in outs:
                for codes, scales in ((o["k_cache"], o["k_scale"]), (o["v_cache"], o["v_scale"])):
                    x = torch.randn(cfg.start_pos, cfg.kv_heads, cfg.head_dim, device=dev, generator=gen).to(torch.bfloat16)
                    Kn.quantize_kv_fp8(codes, scales, x, zero, 1, cfg.start_pos * cfg.kv_heads, cfg.head_dim)

    def forward():
        n = 0
        for l in range(L):
            n += layer_ops.fused_layer_step(cfg, ins[l % n_sets], outs[l % n_sets], with_embedding=(l == 0),
                                            attention_partial=partial)
        return n

    use_graph = args.graph == "on" or (args.graph == "auto" and cfg.tokens == 1)
    launches_per_step = forward()
    torch.cuda.synchronize()
    # Eager steps replay the forward's C-ABI calls as recorded once (same entry points, pointers and stream):
    # what a C++ caller pays per launch, without the Python mirror's argument checks between the launches.
    from runtherder_b200._lib import CallPlan
    with CallPlan() as plan:
        forward()
    torch.cuda.synchronize()
    graph = None
    if use_graph:
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            forward()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                forward()
        torch.cuda.synchronize()
    step = graph.replay if graph is not None else plan.replay

    for _ in range(max(args.warmup, 3)):
        step()
    K = args.steps
    barrier()
    a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clocks:
        a.record()
        for _ in range(K):
            step()
        bb.record()
        torch.cuda.synchronize()
    ms = max_over_ranks(a.elapsed_time(bb)) / K
    barrier()

    peak, peak_kind = measured_peak()
    total_bytes = per_row * T * L + cfg.bytes_embedding() * T
    value = total_bytes / (ms * 1e-3) / 1e9
    line = {"metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32",
            "io_dtypes": "bf16 in; " + ("int8 codes, " if cfg.int8 else "") + "fp8-e4m3 cache bytes, fp32 scales, bf16 out",
            "data": "synthetic", "token_rows_per_s": round(T / (ms * 1e-3), 1), "us_per_layer": round(ms * 1e3 / L, 3),
            "frac_of_hbm_peak": {peak_kind: round(value / (peak * world), 4)},
            "config": {"workload": cfg.name, "token_rows": T, "rows_per_gpu": rows, "layers": L, "hidden": cfg.hidden,
                       "inter": cfg.inter, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                       "int8": cfg.int8, "qk_norm": cfg.qk_norm, "start_pos": cfg.start_pos, "seed": cfg.seed,
                       "ops_per_layer": [n for n, _ in cfg.chain_ops()] + (["attention (flash decode: 2 launches)" if T == 1 else "attention (flash prefill)"] if partial is not None else []),
                       "algorithmic_bytes_per_row_per_layer": per_row,
                       "buffer_sets": n_sets, "cuda_graph": graph is not None,
                       "launch_path": "one CUDA graph" if graph is not None else "recorded C-ABI calls replayed from Python",
                       "parallelism": f"rows/{world}",
                       "l2": f"{n_sets} rotating buffer sets; a set is {'larger' if layer_bytes > 126e6 else 'smaller'} than the 126 MB L2"},
            "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step, "clocks": clocks.summary()}

    # per-kernel roofline from a separate event pass over one layer (not part of the timed region)
    try:
        line["roofline"] = chain_roofline(cfg, ins[0], outs[0], rows, peak, peak_kind)
    except Exception as exc:
        line["roofline"] = {"unavailable": str(exc)[:200]}

    if world == 1 and not args.no_refcuda:
        try:
            line["ref_cuda"] = time_reference_chain(cfg, ins, outs, rows, L, n_sets, total_bytes, use_graph, max(3, min(K, 20)), partial)
        except Exception as exc:
            line["ref_cuda"] = {"unavailable": str(exc)[:200]}
    note_device_error(line)
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_decode_attention(args, cfg, dev, emit=True):
    """Secondary measurement: one decode step's attention per layer — rh_flash_decode_split_bf16 over a
    seeded FP8 cache of `depth` keys, one distinct cache per layer (28 x 16.8 MB at the decode config, more
    than L2), replayed as one CUDA graph like the reference's decode loop.  Algorithmic bytes per call: the K
    and V codes and their scales of every key, once (2*D + 8 bytes per key and kv head)."""
    import math
    import torch
    from runtherder_b200 import kernels as Kn
    depth = args.depth or (cfg.start_pos + 1)
    Hq, Hkv, D, L, S = cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.layers, args.splits
    n_sets = int(min(L, max(2, 3e9 // (depth * Hkv * (2 * D + 8)))))
    gen = torch.Generator(device=dev).manual_seed(cfg.seed + 77)
    at0 = torch.zeros(1, dtype=torch.int32, device=dev)
    sets = []
    for _ in range(n_sets):
        q = torch.randn(Hq, D, device=dev, generator=gen).to(torch.bfloat16)
        kc = torch.empty(depth, Hkv, D, dtype=torch.uint8, device=dev); vc = torch.empty_like(kc)
        ks = torch.empty(depth, Hkv, dtype=torch.float32, device=dev); vs = torch.empty_like(ks)
        for codes, scales in ((kc, ks), (vc, vs)):
            x = torch.randn(depth, Hkv, D, device=dev, generator=gen).to(torch.bfloat16)
            Kn.quantize_kv_fp8(codes, scales, x, at0, 1, depth * Hkv, D)
        sets.append((q, kc, ks, vc, vs))
    cache_len = torch.tensor([depth - 1], dtype=torch.int32, device=dev)
    partial = torch.empty(Kn.flash_split_scratch_floats(Hq, D, S), dtype=torch.float32, device=dev)
    out = torch.empty(Hq, D, dtype=torch.bfloat16, device=dev)
    scale = 1.0 / math.sqrt(D)

    def forward_with(fn):
        for l in range(L):
            q, kc, ks, vc, vs = sets[l % n_sets]
            fn(out, q, kc, vc, ks, vs, partial, S, cache_len, Hq, Hkv, D, scale)

    def timed(fn, reps):
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            forward_with(fn)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                forward_with(fn)
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with ClockSampler(dev.index or 0) as clocks:
            a.record()
            for _ in range(reps):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
        return a.elapsed_time(b) / reps, clocks.summary()

    K = args.steps
    ms, clocks = timed(Kn.flash_decode_split_bf16, K)
    bytes_per_call = depth * Hkv * (2 * D + 8)
    peak, peak_kind = measured_peak()
    achieved = bytes_per_call * L / (ms * 1e-3) / 1e9
    line = {"metric": "flash-decode KV-cache GB/s", "value": round(achieved, 1), "unit": "GB/s", "n_gpus": 1, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "us_per_call": round(ms * 1e3 / L, 2),
            "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "f32",
            "io_dtypes": "bf16 q, fp8-e4m3 cache codes + fp32 scales in; bf16 out (f16 tensor-core operands, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"{cfg.name}: decode attention", "depth": depth, "q_heads": Hq, "kv_heads": Hkv,
                       "head_dim": D, "splits": S, "layers": L, "cache_sets": n_sets, "cuda_graph": True,
                       "algorithmic_bytes_per_call": bytes_per_call,
                       "l2": f"{n_sets} distinct caches of {bytes_per_call / 1e6:.1f} MB replayed in turn"},
            "gpu_launches": 2 * L * K, "launches_per_step": 2 * L, "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "flash_decode_partial + reduce", "achieved": round(achieved, 1),
                         "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                         "traffic": None,
                         "note": "per-call time includes two graph-node launches; short histories are latency-bound"}}
    if not args.no_refcuda:
        try:
            sys.path.insert(0, str(ROOT / "tests"))
            from gpu_util import RefCuda
            ref = RefCuda()

            def ref_fn(out_, q, kc, vc, ks, vs, part, S_, cl, Hq_, Hkv_, D_, sc):
                ref.flash_decode_split_bf16(out_, q, kc, vc, ks, vs, part, S_, cl, Hq_, Hkv_, D_, sc)
            rms, _ = timed(ref_fn, max(3, min(K, 20)))
            line["ref_cuda"] = {"us_per_call": round(rms * 1e3 / L, 2), "value": round(bytes_per_call * L / (rms * 1e-3) / 1e9, 1),
                                "unit": "GB/s (same algorithmic bytes)", "launches_per_step": 2 * L,
                                "what": "reference src/kernels/flash_decode.cu compiled for sm_100a, same caches, same graph replay"}
        except Exception as exc:
            line["ref_cuda"] = {"unavailable": str(exc)[:200]}
    if not args.no_cpu:
        try:
            sys.path.insert(0, str(ROOT / "tests"))
            from gpu_util import to_np
            from oracle_lib import Oracle
            orc = Oracle()
            q, kc, ks, vc, vs = (to_np(t) for t in sets[0])
            t0 = time.perf_counter()
            orc.attention_decode_fp8(q, kc, vc, ks, vs, depth - 1, scale)
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": round(bytes_per_call / dt / 1e9, 4), "unit": "GB/s", "cores": 1, "kind": "port",
                                    "sample": f"one call ({depth} keys, {Hq} heads) of the double-precision oracle, {dt:.2f} s"}
        except Exception as exc:
            line["cpu_baseline"] = {"unavailable": str(exc)[:200]}
    note_device_error(line)
    if emit:
        print(json.dumps(line), flush=True)
    return line


def measured_tensor_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def run_prefill_attention(args, cfg, dev, emit=True):
    """Secondary measurement: the causal prefill attention of one layer — rh_flash_prefill_bf16 on `tokens` new
    tokens over an (initially empty) FP8 cache, a few distinct q/cache sets used in turn.  FLOPs per call:
    4 * head_dim * q_heads * T (T + 1) / 2 (both products, causal half)."""
    import math
    import torch
    from runtherder_b200 import kernels as Kn
    T, Hq, Hkv, D = cfg.tokens, cfg.q_heads, cfg.kv_heads, cfg.head_dim
    n_sets = 3
    gen = torch.Generator(device=dev).manual_seed(cfg.seed + 78)
    at0 = torch.zeros(1, dtype=torch.int32, device=dev)
    sets = []
    for _ in range(n_sets):
        q = torch.randn(T, Hq, D, device=dev, generator=gen).to(torch.bfloat16)
        kc = torch.empty(T, Hkv, D, dtype=torch.uint8, device=dev); vc = torch.empty_like(kc)
        ks = torch.empty(T, Hkv, dtype=torch.float32, device=dev); vs = torch.empty_like(ks)
        for codes, scales in ((kc, ks), (vc, vs)):
            x = torch.randn(T, Hkv, D, device=dev, generator=gen).to(torch.bfloat16)
            Kn.quantize_kv_fp8(codes, scales, x, at0, 1, T * Hkv, D)
        sets.append((q, kc, ks, vc, vs, torch.empty(T, Hq, D, dtype=torch.bfloat16, device=dev)))
    cache_len = torch.zeros(1, dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(D)
    flops = 4.0 * D * Hq * T * (T + 1) / 2

    def timed(fn, reps):
        for i in range(max(args.warmup, 3)):
            fn(*sets[i % n_sets])
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with ClockSampler(dev.index or 0) as clocks:
            a.record()
            for i in range(reps):
                fn(*sets[i % n_sets])
            b.record()
            torch.cuda.synchronize()
        return a.elapsed_time(b) / reps, clocks.summary()

    def ours(q, kc, ks, vc, vs, out):
        Kn.flash_prefill_bf16(out, q, kc, vc, ks, vs, T, cache_len, Hq, Hkv, D, scale)

    K = args.steps
    ms, clocks = timed(ours, K)
    peak, peak_kind = measured_tensor_peak()
    achieved = flops / (ms * 1e-3) / 1e12
    tunes = args.tune or []
    tc_form = not any(t.startswith("prefill_tiles=1") or t.startswith("prefill_tiles=2") for t in tunes)
    parts = [t.split("=", 1)[1] for t in tunes if t.startswith("prefill_parts=")]
    tc_kernel = "flash_prefill_tc_kernel" if parts and parts[-1] in ("1", "2", "3", "4") else "flash_prefill_ws_kernel"
    line = {"metric": "flash-prefill TFLOP/s", "value": round(achieved, 1), "unit": "TFLOP/s", "n_gpus": 1, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32",
            "io_dtypes": "bf16 q, fp8-e4m3 cache codes + fp32 scales in; bf16 out (f16 tensor-core operands, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"{cfg.name}: causal prefill attention, one layer", "tokens": T, "q_heads": Hq,
                       "kv_heads": Hkv, "head_dim": D, "cache_len": 0, "sets": n_sets, "flops_per_call": flops,
                       "l2": "q + out of one call are 2 x %.0f MB; %d sets used in turn" % (T * Hq * D * 2 / 1e6, n_sets)},
            "gpu_launches": K, "launches_per_step": 1, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": tc_kernel if tc_form else "flash_prefill_kernel", "achieved": round(achieved, 1), "peak": peak,
                         "unit": "TFLOP/s", "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": ("tcgen05.mma kernel (S and O in tensor memory); the E4M3->f16 conversion, the per-key scales "
                                  "and the softmax run on the CUDA cores beside it, in warps of their own in the default form") if tc_form else
                                 ("mma.sync kernel: its own ceiling is the legacy tensor path (one m16n8k16 per 8 cycles "
                                  "per SM sub-partition = 576 TFLOP/s at 1.9 GHz), not the tcgen05 figure the peak was measured with")}}
    if not args.no_refcuda:
        try:
            sys.path.insert(0, str(ROOT / "tests"))
            from gpu_util import RefCuda
            ref = RefCuda()

            def theirs(q, kc, ks, vc, vs, out):
                ref.flash_prefill_bf16(out, q, kc, vc, ks, vs, T, cache_len, Hq, Hkv, D, scale)
            rms, _ = timed(theirs, max(2, min(K, 5)))
            line["ref_cuda"] = {"ms_per_step": round(rms, 4), "value": round(flops / (rms * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
                                "what": "reference src/kernels/flash_prefill.cu compiled for sm_100a, same buffers"}
        except Exception as exc:
            line["ref_cuda"] = {"unavailable": str(exc)[:200]}
    if not args.no_cpu:
        try:
            sys.path.insert(0, str(ROOT / "tests"))
            from gpu_util import to_np
            from oracle_lib import Oracle
            orc = Oracle()
            q, kc, ks, vc, vs, _ = sets[0]
            n_s = min(16, T)
            q_s = to_np(q[T - n_s:].contiguous())
            t0 = time.perf_counter()
            orc.attention_causal_fp8(q_s, to_np(kc), to_np(vc), to_np(ks), to_np(vs), T - n_s, scale)
            dt = time.perf_counter() - t0
            fl = 4.0 * D * Hq * sum(T - n_s + t + 1 for t in range(n_s))
            line["cpu_baseline"] = {"value": round(fl / dt / 1e12, 6), "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                    "sample": f"the last {n_s} of {T} tokens through the double-precision oracle, {dt:.2f} s"}
        except Exception as exc:
            line["cpu_baseline"] = {"unavailable": str(exc)[:200]}
    note_device_error(line)
    if emit:
        print(json.dumps(line), flush=True)
    return line


def chain_roofline(cfg, i, o, rows, peak, peak_kind):
    import torch
    from runtherder_b200 import kernels as Kn
    H = cfg.hidden
    if cfg.int8:
        name, bpr = "swiglu_quant", cfg.bytes_swiglu_quant()
        fn = lambda: Kn.swiglu_quant_int8(o["q_mlp"], o["s_mlp"], None, i["gate"], i["up"], rows, cfg.inter)
    else:
        name, bpr = "swiglu", cfg.bytes_swiglu()
        fn = lambda: Kn.swiglu_bf16_forward(o["mlp_act"], i["gate"], i["up"], rows * cfg.inter)
    for _ in range(3):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 20
    achieved = rows * bpr / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}", "traffic": None, "us_per_launch": round(ms * 1e3, 2),
            "note": "back-to-back launches on one buffer set" + ("" if rows * bpr > 126e6 else " that fits in L2: latency-bound, not an HBM figure")}


def time_reference_chain(cfg, ins, outs, rows, L, n_sets, total_bytes, use_graph, reps, partial=None):
    import torch
    sys.path.insert(0, str(ROOT / "tests"))
    from gpu_util import RefCuda
    from runtherder_b200 import layer_ops
    ref = RefCuda()
    scratch = {"normed": torch.empty_like(ins[0]["x"]), "ffn_normed": torch.empty_like(ins[0]["x"]),
               "act": torch.empty_like(ins[0]["gate"])}
    out = {}
    for label, dedup in (("as_issued", False), ("dedup", True)):
        def forward():
            n = 1
            ref.embedding_lookup_bf16_forward(outs[0]["emb"], ins[0]["table"], ins[0]["ids"], rows, cfg.hidden)
            for l in range(L):
                n += layer_ops.reference_sequence(ref, cfg, ins[l % n_sets], outs[l % n_sets], scratch, dedup_quant=dedup,
                                                  attention_partial=partial)
            return n
        with ref.record() as plan:      # eager steps replay the recorded calls, like our own arm's
            n = forward()
        torch.cuda.synchronize()
        step = plan.replay
        if use_graph:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                forward()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    forward()
            torch.cuda.synchronize()
            step = g.replay
        for _ in range(3):
            step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            step()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        out[label] = {"ms_per_step": round(ms, 4), "launches_per_step": n, "value": round(total_bytes / (ms * 1e-3) / 1e9, 1),
                      "unit": "GB/s (same algorithmic bytes)"}
    out["what"] = "reference src/kernels/*.cu compiled for sm_100a through the reference's call sequence, same buffers"
    return out


def time_reference_cuda(cfg, ins, outs, rows, per_row, reps):
    """The reference's kernels (sm_100a build) for the same four ops, as its layer code issues them:
    gather; rmsnorm_add then quantize_per_token_int8 once per consumer GEMM (x3 for q/k/v); rope then two
    quantize_kv_fp8; swiglu then quantize_per_token_int8.  Also timed with the repeated quantisation
    issued once ("dedup")."""
    import torch
    sys.path.insert(0, str(ROOT / "tests"))
    from gpu_util import RefCuda
    ref = RefCuda()
    T, H, I = rows, cfg.hidden, cfg.inter
    normed = torch.empty_like(ins["x"])
    act = torch.empty_like(ins["gate"])

    def seq(n_quant):
        ref.embedding_lookup_bf16_forward(outs["emb"], ins["table"], ins["ids"], T, H)
        ref.rmsnorm_add_bf16_forward(normed, outs["h_attn"], ins["x"], ins["residual"], ins["g_attn"], T, H, cfg.eps)
        for _ in range(n_quant):
            ref.quantize_per_token_int8(outs["q_attn_in"], outs["s_attn_in"], normed, T, H)
        ref.rope_bf16(ins["q"], ins["k"], ins["positions"], ins["inv_freq"], T, cfg.q_heads, cfg.kv_heads, cfg.head_dim)
        ref.quantize_kv_fp8(outs["k_cache"], outs["k_scale"], ins["k"], outs["at_pos"], cfg.kv_heads, T * cfg.kv_heads, cfg.head_dim)
        ref.quantize_kv_fp8(outs["v_cache"], outs["v_scale"], ins["v"], outs["at_pos"], cfg.kv_heads, T * cfg.kv_heads, cfg.head_dim)
        ref.swiglu_bf16_forward(act, ins["gate"], ins["up"], T * I)
        ref.quantize_per_token_int8(outs["q_mlp"], outs["s_mlp"], act, T, I)
        return 7 + n_quant

    k_backup = ins["k"].clone()
    out = {}
    for label, nq in (("as_issued", 3), ("dedup", 1)):
        for _ in range(3):
            n = seq(nq)
        torch.cuda.synchronize()
        a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            seq(nq)
        bb.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(bb) / reps
        out[label] = {"ms_per_step": round(ms, 4), "launches_per_step": n,
                      "value": round(rows * per_row / (ms * 1e-3) / 1e9, 1), "unit": "GB/s (same algorithmic bytes)"}
    ins["k"].copy_(k_backup)
    out["what"] = "reference src/kernels/*.cu compiled for sm_100a, same device buffers, same process"
    return out


def time_end_to_end(cfg, ins, rows, total_bytes, world, barrier, max_over_ranks, steps, dev):
    import torch
    from runtherder_b200 import host_path
    weights = {k: ins[k] for k in ("g_attn", "inv_freq", "table")}
    # at least eight chunks per step, so that the two copy directions and the kernels overlap on small shards too
    chunk_rows = max(512, min(4096, rows // 8))
    runner = host_path.HostSweep(cfg, rows, weights, chunk_rows=chunk_rows, n_slots=3, device=dev)
    host_in = runner.alloc_host_inputs(ins)
    host_out = runner.alloc_host_outputs()
    h2d, d2h = runner.bytes_per_step()
    for _ in range(2):
        runner.run(host_in, host_out)
    barrier()
    t0 = time.perf_counter()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    n = 0
    for _ in range(steps):
        n += runner.run(host_in, host_out)
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = max_over_ranks(max(a.elapsed_time(b), wall * 1e3)) / steps
    barrier()
    h2d_all, d2h_all = max_over_ranks(float(h2d)) * world, max_over_ranks(float(d2h)) * world
    return {"value": round(total_bytes / (ms * 1e-3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(ms, 3),
            "steps": steps, "h2d_bytes_per_step": int(h2d_all), "d2h_bytes_per_step": int(d2h_all),
            "pcie_gbs": {"h2d": round(h2d_all / (ms * 1e-3) / 1e9, 1), "d2h": round(d2h_all / (ms * 1e-3) / 1e9, 1)},
            "launches_per_step": n // steps, "pinned_near_gpu": runner.cpus is not None,
            "chunk_rows": chunk_rows,
            "what": "per chunk of rows: one pinned input record -> one H2D copy -> four fused kernels -> one D2H copy of "
                    "the output record (+ the in-place rotated q); host-to-device, compute and device-to-host each on "
                    "their own stream; bounded by the PCIe link of each GPU"}


if __name__ == "__main__":
    main()
