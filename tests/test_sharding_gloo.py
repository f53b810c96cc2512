"""Row sharding with two CPU ranks over gloo: each rank produces its row block of the layer outputs
(with the oracle standing in for the GPU kernels, which are row-local in the same way), the
verification gather reassembles them, and the result equals the single-rank computation.  A second
case drops one rank before the gather: the survivor's collective ends with an error after a short
process-group timeout instead of hanging."""
import datetime
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_gather(rank, world, port, T, H, result_dir):
    sys.path.insert(0, str(HERE)); sys.path.insert(0, str(HERE.parent))
    from oracle_lib import Oracle
    from refgen import make_bf16_random
    from runtherder_b200.sharding import gather_rows, shard_bounds
    _init(rank, world, port)
    orc = Oracle()
    x = make_bf16_random(T * H, 1.0, 1).reshape(T, H)
    r = make_bf16_random(T * H, 1.0, 2).reshape(T, H)
    g = make_bf16_random(H, 0.5, 3)
    b, e = shard_bounds(T, world, rank)
    y, h = orc.rmsnorm_add(x[b:e].copy(), r[b:e].copy(), g, 1e-5)
    q, s = orc.quant_int8(y)
    full_q = gather_rows(torch.from_numpy(q), T)
    full_s = gather_rows(torch.from_numpy(s), T)
    full_h = gather_rows(torch.from_numpy(h.view(np.int16)), T)
    if rank == 0:
        yy, hh = orc.rmsnorm_add(x, r, g, 1e-5)
        qq, ss = orc.quant_int8(yy)
        ok = (np.array_equal(full_q.numpy(), qq) and np.array_equal(full_s.numpy(), ss)
              and np.array_equal(full_h.numpy().view(np.uint16), hh))
        Path(result_dir, "ok").write_text("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def _worker_window(rank, world, port, T, H, result_dir):
    sys.path.insert(0, str(HERE)); sys.path.insert(0, str(HERE.parent))
    from refgen import make_bf16_random
    from runtherder_b200.sharding import boundary_windows, gather_window, shard_bounds
    _init(rank, world, port)
    full = torch.from_numpy(make_bf16_random(T * H, 1.0, 7).reshape(T, H).view(np.int16)).view(torch.bfloat16)
    scales = torch.arange(T, dtype=torch.float32) + 0.5
    b, e = shard_bounds(T, world, rank)
    ok = True
    windows = boundary_windows(T, world, half_width=5)
    for lo, hi in windows:
        w = gather_window(full[b:e].clone(), T, lo, hi)
        ok = ok and torch.equal(w.view(torch.int16), full[lo:hi].view(torch.int16))
        ws = gather_window(scales[b:e].clone(), T, lo, hi)
        ok = ok and torch.equal(ws, scales[lo:hi])
    covered = set()
    for lo, hi in windows:
        covered.update(range(lo, hi))
    cuts = {0, T - 1} | {c for c in (shard_bounds(T, world, r)[0] for r in range(world))} \
        | {max(0, shard_bounds(T, world, r)[1] - 1) for r in range(world)}
    ok = ok and cuts <= covered
    if rank == 0:
        Path(result_dir, "ok").write_text("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("T,world", [(511, 2), (64, 2), (35, 3)])
def test_boundary_windows_gather_the_owning_ranks_rows(tmp_path, T, world):
    """gather_window (what `bench.py --gpus N` verifies the shards with): every window around a shard
    boundary comes back with each row taken from the rank that owns it, for uneven splits too."""
    port = _free_port()
    mp.spawn(_worker_window, args=(world, port, T, 24, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ok").read_text() == "1"


@pytest.mark.parametrize("T", [511, 64])
def test_two_rank_row_shards_reassemble(tmp_path, T):
    port = _free_port()
    mp.spawn(_worker_gather, args=(2, port, T, 264, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"


def _worker_dropout(rank, world, port, result_dir):
    sys.path.insert(0, str(HERE.parent))
    from runtherder_b200.sharding import gather_rows
    _init(rank, world, port, timeout_s=5)
    dist.barrier()
    if rank == 1:
        Path(result_dir, "left").write_text("1")     # leaves between steps, nothing in flight
        os._exit(0)
    try:
        gather_rows(torch.zeros(4, 8, dtype=torch.int8), 8)
        Path(result_dir, "outcome").write_text("completed")
    except Exception as exc:  # the gloo timeout / connection error
        Path(result_dir, "outcome").write_text("error:" + type(exc).__name__)
    os._exit(0)


def test_missing_rank_ends_the_gather_with_an_error(tmp_path):
    port = _free_port()
    mp.spawn(_worker_dropout, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "left").exists()
    assert (tmp_path / "outcome").read_text().startswith("error:")
