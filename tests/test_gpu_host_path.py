"""The pinned-host driver of the op chain (runtherder_b200.host_path.HostSweep): chunk records in, chunk
records out, three streams.  Its outputs must be the bytes of the same four kernels run once over
device-resident tensors, for row counts that do and do not divide into chunks and for more chunks than
device slots (so every slot is recycled several times)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,chunk,slots", [(700, 256, 3), (512, 128, 2), (35, 4096, 3), (1000, 100, 3)])
def test_host_sweep_equals_device_resident_step(rows, chunk, slots):
    from gpu_util import bits_equal
    from runtherder_b200 import host_path, layer_ops, synth
    from runtherder_b200.configs import C0
    cfg = C0.with_tokens(rows)
    ins = synth.make_inputs(cfg, rows=rows)
    weights = {k: ins[k] for k in ("g_attn", "inv_freq", "table")}
    runner = host_path.HostSweep(cfg, rows, weights, chunk_rows=chunk, n_slots=slots)
    host_in = runner.alloc_host_inputs(ins)
    host_out = runner.alloc_host_outputs()
    h2d, d2h = runner.bytes_per_step()
    assert h2d == rows * (2 * (2 * cfg.hidden + cfg.q_dim + 2 * cfg.kv_dim + 2 * cfg.inter) + 8)
    for _ in range(2):                                  # twice: the second pass recycles every slot and event
        launches = runner.run(host_in, host_out)
        torch.cuda.synchronize()
    assert launches == 4 * runner.n_chunks
    got = runner.unpack_outputs(host_out)
    outs = layer_ops.alloc_outputs(cfg, rows, slots=rows)
    host_path.sweep_step(cfg, ins, outs)                # rotates ins["q"] in place
    torch.cuda.synchronize()
    outs["q_rot"] = ins["q"]
    for name, t in got.items():
        assert bits_equal(t.cuda(), outs[name]), name
