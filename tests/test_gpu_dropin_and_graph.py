"""(1) The reference's unmodified kernel tests, compiled against this library through the reference's own
C++ signatures (oracle/_ref/dropin_test_*), must pass.  (2) The fused chain must be capturable in a CUDA
graph and pick up new positions / write slots on replay, as the reference's decode loop requires
(src/engine/generator.cu:46-68: pointers frozen, contents of positions and at_pos change)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("suite", ["rmsnorm", "quantization", "rope", "activation", "bias", "flash_decode", "flash_prefill"])
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
    assert after.value == 0                                                        # the sticky word is not the probe's
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0                                            # context still usable


def test_role_wait_gives_up_raises_the_flag_and_releases_the_other_role():
    """The waits between the warp roles of the prefill attention kernel: a wait that nothing completes runs
    out after its limit and raises the CTA-wide flag; another role, waiting with the kernel's own limit of 2^20
    tries, is released by the flag at once; the kernel returns normally and the context keeps working."""
    import ctypes as C
    from runtherder_b200 import _lib
    result = (C.c_int * 4)(-1, -1, -1, -1)
    _lib.call("rh_selfcheck_role_wait", 64, result)
    claimed, flag, err, other_tries = list(result)
    assert claimed == 0 and flag == 1
    assert err != 0 and (err & 0xff) == 1 and (err >> 8) > 0                       # (source line << 8) | code
    assert 0 < other_tries < 4096                                                  # released by the flag, not by its own 2^20
    after = C.c_int(-1)
    _lib.call("rh_device_error", C.byref(after))
    assert after.value == 0                                                        # the sticky word is not the probe's
    with pytest.raises(_lib.RhError):
        _lib.call("rh_selfcheck_role_wait", 8, result)
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0                                            # context still usable


def test_decode_glue_advances_positions_inside_a_graph():
    """rh_stage_positions == iota + decode_pos copy; rh_decode_advance captured at the end of a step makes
    every replay of the graph see the next position and the previously sampled token, with no host copy."""
    from runtherder_b200 import kernels as K
    positions = torch.full((40,), -1, dtype=torch.int32, device="cuda")
    decode_pos = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    K.stage_positions(positions, decode_pos, 17, 35)
    assert positions[:35].tolist() == list(range(17, 52)) and positions[35:].tolist() == [-1] * 5
    assert decode_pos.item() == 17
    token = torch.tensor([5], dtype=torch.int32, device="cuda")
    sampled = torch.tensor([0], dtype=torch.int32, device="cuda")
    pos1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.stage_positions(pos1, decode_pos, 100, 1)
    seen = torch.zeros(4, 3, dtype=torch.int32, device="cuda")
    step_idx = torch.zeros(1, dtype=torch.int64, device="cuda")
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            row = torch.stack([token[0], pos1[0], decode_pos[0]])      # what a forward would read this step
            seen.index_copy_(0, step_idx, row.unsqueeze(0))
            sampled.copy_(token + 7)                                   # stand-in for the sampler
            K.decode_advance(token, pos1, decode_pos, sampled, 1)
            step_idx.add_(1)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    assert seen.tolist() == [[5, 100, 100], [12, 101, 101], [19, 102, 102], [26, 103, 103]]


def test_dependent_launch_keeps_stream_order_for_device_scalars_and_in_place_chains():
    """Kernels are launched so that each may be scheduled while its predecessor drains and orders itself
    on the device.  A captured run of 64 steps [append a KV row at *at_pos; advance *at_pos] (read-after-
    write on the scalar, kernel to kernel) and an in-place chain rmsnorm_add -> swiglu -> quantise on
    shared buffers (write-after-read) must give exactly the bytes of the same calls launched without the
    attribute and with a synchronise between them."""
    from gpu_util import bits_equal
    from runtherder_b200 import kernels as K
    steps, hkv, d, hidden = 64, 8, 128, 1024
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(steps, hkv * d, device="cuda", generator=gen).to(torch.bfloat16)
    at_pos = torch.zeros(1, dtype=torch.int32, device="cuda")

    def append_all(sync):
        cache = torch.zeros(steps + 2, hkv, d, dtype=torch.uint8, device="cuda")
        scale = torch.zeros(steps + 2, hkv, dtype=torch.float32, device="cuda")
        at_pos.fill_(1)
        for s in range(steps):
            K.quantize_kv_fp8(cache, scale, x[s], at_pos, hkv, hkv, d)
            K.decode_advance(None, None, at_pos, None, 1)
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return cache, scale

    K.tune("no_pdl", 1)
    want_cache, want_scale = append_all(sync=True)
    K.tune("no_pdl", 0)
    got_cache, got_scale = append_all(sync=False)
    assert at_pos.item() == 1 + steps
    assert bits_equal(got_cache, want_cache) and bits_equal(got_scale, want_scale)
    assert bool((want_scale[1:steps + 1] > 0).all()) and bool((want_scale[0] == 0).all())

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    cache = torch.zeros_like(want_cache)
    scale = torch.zeros_like(want_scale)
    with torch.cuda.stream(side):
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for s in range(steps):
                K.quantize_kv_fp8(cache, scale, x[s], at_pos, hkv, hkv, d)
                K.decode_advance(None, None, at_pos, None, 1)
    at_pos.fill_(1)
    graph.replay()
    torch.cuda.synchronize()
    assert bits_equal(cache, want_cache) and bits_equal(scale, want_scale)

    rows = 300
    h0 = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    mlp = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.randn(hidden, device="cuda", generator=gen).to(torch.bfloat16)

    def chain(sync):
        h, y, t = h0.clone(), torch.empty_like(h0), mlp.clone()
        q = torch.empty(rows, hidden, dtype=torch.int8, device="cuda")
        qs = torch.empty(rows, dtype=torch.float32, device="cuda")
        for _ in range(6):
            K.rmsnorm_add_bf16_forward(y, h, t, h, g, rows, hidden, 1e-5)      # h updated in place, y written
            if sync: torch.cuda.synchronize()
            K.swiglu_bf16_forward(t, y, t, rows * hidden)                      # t overwritten from y and itself
            if sync: torch.cuda.synchronize()
            K.quantize_per_token_int8(q, qs, t, rows, hidden)
            if sync: torch.cuda.synchronize()
        torch.cuda.synchronize()
        return h, y, t, q, qs

    K.tune("no_pdl", 1)
    want = chain(sync=True)
    K.tune("no_pdl", 0)
    got = chain(sync=False)
    for a, b in zip(got, want):
        assert bits_equal(a, b)


_FIRST_USE_IN_CAPTURE = r"""
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import torch
from gpu_util import bits_equal
from runtherder_b200 import kernels as K, layer_ops, synth
from runtherder_b200.configs import C0, C3
torch.cuda.set_device(0)
K.init(0)                      # nothing of the library has run yet in this process
for cfg in (C0, C3.with_tokens(700)):
    T = cfg.tokens
    ins = synth.make_inputs(cfg)                       # the generators are not part of the captured path
    q0 = ins["q"].clone()
    outs = layer_ops.alloc_outputs(cfg, T, slots=T)
    last = torch.empty(cfg.hidden, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):     # first use of every kernel below is inside this capture
            layer_ops.fused_layer_step(cfg, ins, outs, with_embedding=True)
            K.rmsnorm_add_last_row(last, ins["x"], ins["residual"], ins["g_ffn"], T, cfg.hidden, cfg.eps)
    graph.replay()
    torch.cuda.synchronize()
    got = {{k: v.clone() for k, v in outs.items()}}
    got["q"], got["last"] = ins["q"].clone(), last.clone()
    ins["q"].copy_(q0)
    outs2 = layer_ops.alloc_outputs(cfg, T, slots=T)
    layer_ops.fused_layer_step(cfg, ins, outs2, with_embedding=True)     # the same calls, eagerly
    K.rmsnorm_add_last_row(last, ins["x"], ins["residual"], ins["g_ffn"], T, cfg.hidden, cfg.eps)
    torch.cuda.synchronize()
    outs2["q"], outs2["last"] = ins["q"], last
    for k, v in got.items():
        if v.dtype.is_floating_point or v.dtype in (torch.int8, torch.uint8):
            assert bits_equal(v, outs2[k]), (cfg.name, k)
print("FIRST-USE-IN-CAPTURE-OK")
"""


def test_first_use_of_every_kernel_inside_capture_after_rh_init():
    """A fresh process calls rh_init and then records a layer's whole chain into a CUDA graph as the very
    first use of the library: no kernel has set-up left to do inside the capture, and the replay produces
    the bytes of the eager calls."""
    code = _FIRST_USE_IN_CAPTURE.format(root=str(ROOT), tests=str(ROOT / "tests"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FIRST-USE-IN-CAPTURE-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("T,H", [(35, 3072), (511, 3072), (1, 4096), (700, 4096), (9, 264)])
def test_final_norm_of_the_last_row_only(T, H):
    """rh_rmsnorm_add_last_row_bf16 == row T-1 of rmsnorm_add_bf16_forward (the reference's final norm,
    llama3.cu:254-263), bit for bit, against the reference's own kernel; the inputs are left untouched."""
    from gpu_util import bits_equal, ref_cuda_or_skip, to_dev
    from refgen import make_bf16_random
    from runtherder_b200 import kernels as K
    ref = ref_cuda_or_skip()
    x = to_dev(make_bf16_random(T * H, 1.0, 41)).view(T, H)
    r = to_dev(make_bf16_random(T * H, 1.0, 42)).view(T, H)
    g = to_dev(make_bf16_random(H, 1.0, 43))
    x0, r0 = x.clone(), r.clone()
    y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda"); h = torch.empty_like(y)
    ref.rmsnorm_add_bf16_forward(y, h, x, r, g, T, H, 1e-5)
    last = torch.full((H,), 7.0, dtype=torch.bfloat16, device="cuda")
    K.rmsnorm_add_last_row(last, x, r, g, T, H, 1e-5)
    torch.cuda.synchronize()
    assert bits_equal(last, y[T - 1])
    assert bits_equal(x, x0) and bits_equal(r, r0)
