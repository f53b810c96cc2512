"""(1) The reference's unmodified kernel tests, compiled against this library through the reference's own
C++ signatures (oracle/_ref/dropin_test_*), must pass.  (2) The fused chain must be capturable in a CUDA
graph and pick up new positions / write slots on replay, as the reference's decode loop requires
(src/engine/generator.cu:46-68: pointers frozen, contents of positions and at_pos change)."""
import subprocess
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("suite", ["rmsnorm", "quantization", "rope", "activation"])
def test_reference_kernel_tests_pass_against_this_library(suite):
    exe = ROOT / "oracle" / "_ref" / f"dropin_test_{suite}"
    if not exe.exists():
        pytest.skip(f"{exe.name} was not built (needs the reference sources at build time)")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "0 failed expectations" in r.stdout


def test_decode_chain_in_cuda_graph_tracks_position():
    from gpu_util import bits_equal
    from runtherder_b200 import layer_ops, synth
    from runtherder_b200.configs import C2
    cfg = C2
    layers = 4
    ins = [synth.make_inputs(cfg.with_tokens(1), rows=1, row_offset=l, with_table=(l == 0)) for l in range(layers)]
    outs = [layer_ops.alloc_outputs(cfg, 1, slots=cfg.cache_slots) for _ in range(layers)]
    at_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    positions = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_orig = [i["q"].clone() for i in ins]
    for i, o in zip(ins, outs):
        i["positions"], o["at_pos"] = positions, at_pos

    def forward(stream=None):
        n = 0
        for l, (i, o) in enumerate(zip(ins, outs)):
            n += layer_ops.fused_layer_step(cfg, i, o, stream=stream, with_embedding=(l == 0))
        return n

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        forward()                                     # first step eagerly, like the reference
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            launches = forward()
    assert launches == 1 + 5 * layers

    for pos in (8195, 17, 4000):
        for i, q0 in zip(ins, q_orig):
            i["q"].copy_(q0)
        positions.fill_(pos); at_pos.fill_(pos)
        graph.replay()
        torch.cuda.synchronize()
        got = [(o["k_cache"][pos].clone(), o["k_scale"][pos].clone(), i["q"].clone(), o["q_mlp"].clone()) for i, o in zip(ins, outs)]
        for i, q0 in zip(ins, q_orig):
            i["q"].copy_(q0)
        for o in outs:
            o["k_cache"][pos].zero_(); o["k_scale"][pos].zero_()
        forward()
        torch.cuda.synchronize()
        for (kc, ks, q, qm), i, o in zip(got, ins, outs):
            assert bits_equal(kc, o["k_cache"][pos]) and bits_equal(ks, o["k_scale"][pos])
            assert bits_equal(q, i["q"]) and bits_equal(qm, o["q_mlp"])
            assert bool(o["k_scale"][pos].abs().sum() > 0)


def test_bounded_wait_gives_up_and_reports():
    """Failure detection without a fault: a wait on a barrier nothing completes runs out after its poll
    limit, the kernel returns normally, the error word says where, and the context keeps working."""
    import ctypes as C
    from runtherder_b200 import _lib
    gave_up, err = C.c_int(-1), C.c_int(-1)
    _lib.call("rh_selfcheck_bounded_wait", 64, C.byref(gave_up), C.byref(err))
    assert gave_up.value == 1
    assert err.value != 0 and (err.value & 0xff) == 1 and (err.value >> 8) > 0    # (source line << 8) | code
    after = C.c_int(-1)
    _lib.call("rh_device_error", C.byref(after))
    assert after.value == 0                                                        # sticky word restored
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0                                            # context still usable
