"""Host-side logic that needs no GPU: argument validation of the C ABI (every check happens before any
CUDA call), the Python mirror's checks, frequency tables, configuration byte counts, row sharding."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle_lib import Oracle
from runtherder_b200 import _lib, kernels as K
from runtherder_b200.configs import C0, C1, C2, C3, C4, CONFIGS, RopeScaling
from runtherder_b200.rope_tables import inv_freq_for, rope_inv_freq_llama3, rope_inv_freq_plain
from runtherder_b200.sharding import all_shard_bounds, shard_bounds
from runtherder_b200.synth import outlier_channel_scale

ORC = Oracle()
A = 0x7f0000000000  # a 16-byte-aligned, never dereferenced device address


def status(name, *args):
    return getattr(_lib.lib, name)(*args)


def test_capi_rejects_bad_arguments_before_launching():
    L = _lib
    # rmsnorm: the reference's checks (src/kernels/rmsnorm.cu:170-179, 205-208)
    assert status("rh_rmsnorm_bf16", A, A, A, 0, 128, 1e-5, None) == 1
    assert status("rh_rmsnorm_bf16", A, A, A, 4, 4, 1e-5, None) == 2
    assert status("rh_rmsnorm_bf16", A, A, A, 4, 12, 1e-5, None) == 2
    assert status("rh_rmsnorm_bf16", A, A, A, 4, 16392, 1e-5, None) == 2
    assert status("rh_rmsnorm_bf16", A, A, A, 4, 128, 0.0, None) == 1
    assert status("rh_rmsnorm_bf16", A, None, A, 4, 128, 1e-5, None) == 1
    assert status("rh_rmsnorm_bf16", A + 2, A, A, 4, 128, 1e-5, None) == 3
    assert status("rh_rmsnorm_add_bf16", A, A, A, A, A, 4, 128, 1e-5, None) == 1      # y == h_out
    assert b"distinct" in L.lib.rh_last_error_string()
    # int8 / fp8 quantisation (quantization.cu:122-124, 280-284)
    assert status("rh_quantize_per_token_int8", A, A, A, 0, 128, None) == 1
    assert status("rh_quantize_per_token_int8", A, A, A, 2, 20, None) == 2
    assert status("rh_quantize_kv_fp8", A, A, A, None, 8, 16, 128, None) == 1         # at_pos null
    assert status("rh_quantize_kv_fp8", A, A, A, A, 0, 16, 128, None) == 1            # rows_per_pos
    assert status("rh_quantize_kv_fp8", A, A, A, A, 8, 16, 12, None) == 2
    # swiglu (activation.cu:50-51)
    assert status("rh_swiglu_bf16", A, A, A, 4, None) == 2
    assert status("rh_swiglu_bf16", A, A, A, 12, None) == 2
    assert status("rh_swiglu_quant_int8", A, A, None, A, A, 4, 20000, None) == 2
    # rope (rope.cu:69-74)
    assert status("rh_rope_bf16", A, A, A, A, 0, 4, 1, 64, None) == 1
    assert status("rh_rope_bf16", A, A, A, A, 1, 4, 1, 7, None) == 2
    assert status("rh_rope_bf16", A, A, A, A, 1, 4, 1, 258, None) == 2
    assert status("rh_rope_kv_fp8", A, None, A, A, None, None, 1e-6, A, A, A, A, A, A, A, 1, 4, 1, 24, None) == 2
    assert status("rh_rope_kv_fp8", A, None, A, A, A, None, 1e-6, A, A, A, A, A, A, A, 1, 4, 1, 128, None) == 1
    assert status("rh_rope_kv_fp8", A, None, A, A, None, None, 1e-6, A, A, A, A, A, A, None, 1, 4, 1, 128, None) == 1
    # embedding (embedding.cu:47-49), epilogue (quantization.cu:183-184)
    assert status("rh_embedding_lookup_bf16", A, A, A, 0, 128, None) == 1
    assert status("rh_embedding_lookup_bf16", A, A, A, 3, 12, None) == 2
    assert status("rh_dequantize_w8a8", A, A, A, A, 0, 5, None) == 1
    assert status("rh_tune", b"no_such_knob", 3) == 1
    assert status("rh_tune", b"rows_ctas_per_sm", 0) == 0
    # attention over the FP8 cache (flash_decode.cu:288-293, flash_prefill.cu:227-229) and the bias-fused RoPE+KV
    assert status("rh_flash_decode_split_bf16", A, A, A, A, A, A, A, 0, A, 8, 2, 128, 0.1, None) == 1      # num_splits
    assert status("rh_flash_decode_split_bf16", A, A, A, A, A, A, A, 4, None, 8, 2, 128, 0.1, None) == 1   # cache_len null
    assert status("rh_flash_decode_split_bf16", A, A, A, A, A, A, A, 4, A, 8, 3, 128, 0.1, None) == 1      # 8 % 3
    assert status("rh_flash_decode_split_bf16", A, A, A, A, A, A, A, 4, A, 8, 2, 1024, 0.1, None) == 2
    assert status("rh_flash_decode_split_bf16", A, A + 2, A, A, A, A, A, 4, A, 8, 2, 128, 0.1, None) == 3
    assert L.lib.rh_flash_split_scratch_floats(32, 128, 32) == 32 * 32 * 130
    assert status("rh_flash_prefill_bf16", A, A, A, A, A, A, 0, A, 8, 2, 128, 0.1, None) == 1              # n_new
    assert status("rh_flash_prefill_bf16", A, A, A, A, A, A, 4, A, 8, 2, 64, 0.1, None) == 2
    assert b"128" in L.lib.rh_last_error_string()
    assert status("rh_flash_prefill_bf16", A, A, A, A, None, A, 4, A, 8, 2, 128, 0.1, None) == 1
    assert status("rh_bias_rope_kv_fp8", A, None, A, A, A, A, None, A, A, A, A, A, A, A, 1, 4, 1, 128, None) == 1   # a bias missing
    assert status("rh_bias_rope_kv_fp8", A, None, A, A, A, A, A, A, A, A, A, A, A, A, 1, 4, 1, 48, None) == 2
    assert status("rh_tune", b"prefill_tiles", 0) == 0 and status("rh_tune", b"no_pdl", 0) == 0


def test_python_mirror_raises_like_the_reference_exits():
    cpu = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(K.RhError):
        K.rmsnorm_bf16_forward(cpu, cpu, cpu[0], 4, 128, 1e-5)           # not a CUDA tensor
    with pytest.raises(K.RhError) as e:
        K.rmsnorm_bf16_forward(A, A, A, 4, 100, 1e-5, stream=0)
    assert e.value.status == 2 and "divisible by 8" in str(e.value)
    with pytest.raises(K.RhError):
        K.quantize_kv_fp8(A, A, A, None, 8, 8, 128, stream=0)


def test_inv_freq_tables():
    assert np.array_equal(rope_inv_freq_plain(128, 1.0e6).view(np.uint32), ORC.inv_freq_plain(128, 1.0e6).view(np.uint32))
    a = rope_inv_freq_llama3(128, 500000.0, RopeScaling())
    assert np.array_equal(a.view(np.uint32), ORC.inv_freq_llama3(128, 500000.0, 32.0, 1.0, 4.0, 8192).view(np.uint32))
    assert hex(a.view(np.uint32)[32]) == "0x39e13623"
    assert np.array_equal(inv_freq_for(C3), rope_inv_freq_plain(128, 1.0e6))
    assert np.array_equal(inv_freq_for(C4), a)
    out = (C.c_float * 4)()
    assert status("rh_rope_inv_freq_plain", out, 7, 1e4) == 2
    assert status("rh_rope_inv_freq_plain", out, 8, -1.0) == 1
    assert status("rh_rope_inv_freq_plain", None, 8, 1e4) == 1


def test_config_byte_counts():
    assert C0.bytes_rope_kv() == 18500 and C4.bytes_rope_kv() == 22596
    assert C4.bytes_norm_quant() == 7 * 4096 + 4 and C4.bytes_swiglu_quant() == 5 * 14336 + 4
    assert C3.bytes_norm() == 8 * 4096 and C3.bytes_swiglu() == 6 * 12288
    assert C4.bytes_embedding() == 4 * 4096 + 4 and C4.bytes_quant(C4.q_dim) == 3 * 4096 + 4
    assert round(C4.tokens * C4.bytes_norm_quant() / 1e9, 3) == 1.879
    assert round(C4.tokens * C4.bytes_swiglu_quant() / 1e9, 3) == 4.698
    assert round(C4.tokens * C4.bytes_rope_kv() / 1e9, 3) == 1.481
    assert [n for n, _ in C1.chain_ops()] == ["norm_quant", "rope_kv", "quant_attn", "norm_quant", "swiglu_quant"]
    assert [n for n, _ in C3.chain_ops()] == ["norm", "rope_kv", "norm", "swiglu"]
    assert C2.start_pos == 8195 and C2.cache_slots == 8196 and C1.cache_slots == 511
    assert set(CONFIGS) == {"c0", "c1", "c2", "c3", "c4"}


def test_outlier_channels():
    for H, n in [(3072, 16), (4096, 21)]:
        s = outlier_channel_scale(H, 0, 1)
        assert (s == 20.0).sum() == n and (s == 1.0).sum() == H - n
        assert np.array_equal(s, outlier_channel_scale(H, 0, 1))
        assert not np.array_equal(s, outlier_channel_scale(H, 1, 1))


def test_shard_bounds_cover_rows_contiguously():
    for T in (1, 35, 511, 8192, 65536):
        for G in (1, 2, 4, 8):
            b = all_shard_bounds(T, G)
            assert b[0][0] == 0 and b[-1][1] == T
            assert all(b[i][1] == b[i + 1][0] for i in range(G - 1))
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(sizes) <= 1
    assert shard_bounds(511, 2, 0) == (0, 255) and shard_bounds(511, 2, 1) == (255, 511)
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def test_row_locality_of_the_oracle():
    """Every op is row-local: computing a shard alone gives the same rows as computing everything —
    the property row sharding rests on.  Checked on the oracle here; on the kernels in the GPU tests."""
    from refgen import make_bf16_random
    T, H = 22, 256
    x, r = make_bf16_random(T * H, 1.0, 1).reshape(T, H), make_bf16_random(T * H, 1.0, 2).reshape(T, H)
    g = make_bf16_random(H, 0.5, 3)
    y, h = ORC.rmsnorm_add(x, r, g, 1e-5)
    q, s = ORC.quant_int8(y)
    for b, e in all_shard_bounds(T, 4):
        ys, hs = ORC.rmsnorm_add(x[b:e].copy(), r[b:e].copy(), g, 1e-5)
        qs, ss = ORC.quant_int8(ys)
        assert np.array_equal(ys, y[b:e]) and np.array_equal(hs, h[b:e])
        assert np.array_equal(qs, q[b:e]) and np.array_equal(ss, s[b:e])


def test_new_entry_points_reject_bad_arguments_before_launching():
    # final norm of the last row, rh_init, the W8A8 linear wrapper (matmul.cu:135-136)
    assert status("rh_rmsnorm_add_last_row_bf16", A, A, A, A, 0, 128, 1e-5, None) == 1
    assert status("rh_rmsnorm_add_last_row_bf16", A, A, A, A, 4, 12, 1e-5, None) == 2
    assert status("rh_rmsnorm_add_last_row_bf16", A, A, None, A, 4, 128, 1e-5, None) == 1
    assert status("rh_rmsnorm_add_last_row_bf16", A, A + 8, A, A, 4, 128, 1e-5, None) == 3
    assert status("rh_init", -1) != 0                       # no such device (and no device at all on a CPU box)
    from runtherder_b200 import linear
    call = linear.lib.rh_linear_w8a8_prequantized
    assert call(A, A, A, A, A, A, 4, 8, 6, A, None, 0, None) == 2     # k % 4
    assert call(A, A, A, A, A, A, 0, 8, 8, A, None, 0, None) == 1     # m
    assert call(A, A, A, A, A, A, 4, 8, 8, None, None, 0, None) == 1  # no cuBLASLt handle
    assert call(A, A, A, A, A, A, 4, 8, 8, A, None, 64, None) == 1    # workspace size without a workspace
    assert linear.lib.rh_linear_w8a8(A, None, A, A, A, A, A, 4, 8, 8, A, None, 0, None) == 1
    assert linear.lib.rh_linear_release(None) == 1


def test_boundary_windows_cover_every_cut():
    from runtherder_b200.sharding import boundary_windows
    for T, world, half in ((65536, 8, 64), (511, 8, 64), (511, 2, 5), (35, 3, 4), (8, 8, 64)):
        wins = boundary_windows(T, world, half)
        assert all(0 <= lo < hi <= T for lo, hi in wins)
        assert all(a[1] < b[0] for a, b in zip(wins, wins[1:]))           # disjoint, ordered, merged
        covered = set()
        for lo, hi in wins:
            covered.update(range(lo, hi))
        for b, e in all_shard_bounds(T, world):
            if e > b:
                assert b in covered and e - 1 in covered
        assert 0 in covered and T - 1 in covered
    assert boundary_windows(65536, 8, 64)[0] == (0, 64) and len(boundary_windows(65536, 8, 64)) == 9


def test_host_record_layout():
    """The chunk records of the pinned-host driver: fields 256-byte aligned, no overlap, payload = sum of fields."""
    from runtherder_b200.host_path import _Record
    rec = _Record([("x", (3072,), torch.bfloat16), ("ids", (), torch.int32), ("q", (24, 128), torch.bfloat16),
                   ("codes", (3072,), torch.int8), ("s", (), torch.float32)], rows=100)
    spans = []
    for name, (off, shape, dtype) in rec.fields.items():
        n = int(np.prod(shape)) * torch.tensor([], dtype=dtype).element_size()
        assert off % 256 == 0 and shape[0] == 100
        spans.append((off, off + n))
    spans.sort()
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= rec.nbytes
    assert rec.payload == 100 * (3072 * 2 + 4 + 24 * 128 * 2 + 3072 + 4)
    block = torch.zeros(rec.nbytes, dtype=torch.uint8)
    v = rec.views(block, 7)
    assert v["q"].shape == (7, 24, 128) and v["ids"].shape == (7,) and v["codes"].dtype == torch.int8
    v["ids"][:] = torch.arange(7, dtype=torch.int32)
    assert rec.views(block)["ids"][:7].tolist() == list(range(7))         # views alias the block


def test_call_plan_records_and_replays_c_abi_calls():
    """_lib.CallPlan: calls made inside the block are executed and recorded; replay issues them again with
    the same arguments; a failing call raises on replay as it does live."""
    with _lib.CallPlan() as plan:
        _lib.call("rh_tune", b"rows_ctas_per_sm", 3)
        _lib.call("rh_tune", b"rows_ctas_per_sm", 0)
    assert [name for _, name, _ in plan.calls] == ["rh_tune", "rh_tune"]
    assert plan.replay() == 2
    _lib.call("rh_tune", b"rows_ctas_per_sm", 0)                 # nothing is recorded outside the block
    assert len(plan.calls) == 2
    bad = _lib.CallPlan()
    bad.calls.append((_lib.lib.rh_tune, "rh_tune", (b"no_such_knob", 1)))
    with pytest.raises(_lib.RhError):
        bad.replay()
    with _lib.CallPlan():
        with pytest.raises(RuntimeError):
            with _lib.CallPlan():
                pass


def test_reference_call_plan_records_through_a_stand_in_library():
    """gpu_util.RefCuda.record(): calls go to the real library and are replayed with the same arguments."""
    import gpu_util

    class FakeLib:
        def __init__(self):
            self.seen = []

        def refcuda_swiglu(self, *args):
            self.seen.append(args)

    owner = gpu_util.RefCuda.__new__(gpu_util.RefCuda)
    owner.lib = owner._real_lib = FakeLib()
    with owner.record() as plan:
        owner.lib.refcuda_swiglu(1, 2, 3, 4, None)
    assert owner.lib is owner._real_lib
    owner.lib.refcuda_swiglu(9, 9, 9, 9, None)       # not recorded
    assert plan.replay() == 1
    assert owner._real_lib.seen == [(1, 2, 3, 4, None), (9, 9, 9, 9, None), (1, 2, 3, 4, None)]
