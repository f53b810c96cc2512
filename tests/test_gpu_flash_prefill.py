"""Causal prefill attention over the FP8 cache (rh_flash_prefill_bf16) against the double-precision oracle
and the reference's own CUDA kernels (naive attention — the oracle of tests/kernels/test_flash_prefill.cpp —
and flash_prefill_bf16), on the reference test's five shapes and larger / raggeder ones.

Tolerance (floating point): every output within ONE bf16 ulp of the correctly rounded exact value wherever
|exact| >= row max / 16, and within 1.5 * 2^-7 of the row maximum everywhere (one ulp at the row's scale).
The softmax weights enter the second tensor-core product as single f16 values, as in the reference's kernel
(include/runtherder/kernels/flash_prefill.cuh:21-24), so elements that are small against their row carry the
2^-12 rounding of the large terms: measured here at most 4 ulp at row max / 64.  The reference's flash kernel,
which also rounds K*scale and V*scale to f16, reaches 25 ulp there and 2-8 ulp at row max / 16; its test's own
acceptance (max-abs 5e-2, cosine 0.998 against the naive kernel, tests/kernels/test_flash_prefill.cpp:88-89)
is asserted as well, and the reference's naive fp32 kernel is held to the one-ulp bar at row max / 64, which
pins the oracle."""
import math

import numpy as np
import pytest
import torch

from gpu_util import ref_cuda_or_skip, to_np
from oracle_lib import Oracle
from test_gpu_flash_decode import ROWMAX_TOL, ULP_TOL, ordered

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def orc():
    return Oracle()


@pytest.fixture(scope="module")
def ref():
    try:
        return ref_cuda_or_skip()
    except RuntimeError as exc:
        pytest.skip(str(exc))


def make_case(n_new, cache_len, Hq, Hkv, D, seed, q_mul=1.0, dist="uniform", v_spread=0.0):
    from runtherder_b200 import kernels as K
    g = torch.Generator(device="cuda").manual_seed(seed)
    n = cache_len + n_new
    if dist == "uniform":
        q = (torch.rand(n_new, Hq, D, device="cuda", generator=g) * 2 - 1) * q_mul
        k = torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1
        v = torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1
    else:
        q = torch.randn(n_new, Hq, D, device="cuda", generator=g) * q_mul
        k = torch.randn(n, Hkv, D, device="cuda", generator=g)
        v = torch.randn(n, Hkv, D, device="cuda", generator=g)
    if v_spread:
        v = v * torch.exp(torch.randn(n, Hkv, 1, device="cuda", generator=g) * v_spread)
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    at = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda"); vc = torch.empty_like(kc)
    ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda"); vs = torch.empty_like(ks)
    K.quantize_kv_fp8(kc, ks, k, at, 1, n * Hkv, D)
    K.quantize_kv_fp8(vc, vs, v, at, 1, n * Hkv, D)
    return q, kc, ks, vc, vs


def check(out, exact_bits, exact, what, significance=16):
    got_bits, got = to_np(out), out.float().cpu().numpy()
    assert np.isfinite(got).all(), what
    rowmax = np.abs(exact).max(axis=-1, keepdims=True)
    err = np.abs(got - exact)
    assert (err <= ROWMAX_TOL * rowmax + 1e-30).all(), (what, float((err / rowmax).max()))
    significant = np.abs(exact) >= rowmax / significance
    ulp = np.abs(ordered(got_bits) - ordered(exact_bits))
    assert ulp[significant].max(initial=0) <= ULP_TOL, (what, int(ulp[significant].max()))


REFERENCE_TEST_CASES = [(16, 0, 32, 8), (20, 0, 32, 8), (8, 10, 32, 8), (64, 0, 24, 8), (3, 0, 8, 2)]
MORE_CASES = [
    (511, 0, 24, 8),      # the prefill configuration's length (Llama-3.2-3B, three heads per kv head)
    (200, 300, 32, 8),    # chunked prefill behind 300 cached keys
    (130, 63, 28, 4),     # seven heads per kv head, diagonal off the tile grid
    (97, 1, 16, 1),       # sixteen heads on one kv head: two head chunks
    (129, 0, 2, 2),       # no grouping: eight 16-token sub-tiles per CTA
    (1, 77, 8, 2),        # a single token (the decode shape through the prefill entry)
    (97, 31, 8, 4),       # two heads per kv head: 64 tokens x 2 heads per 128-row tile
    (70, 200, 16, 2),     # eight heads per kv head: two head chunks of four
    (33, 5, 10, 2),       # five heads per kv head: a full chunk and a chunk with one live head slot
]


@pytest.mark.parametrize("n_new,cache_len,Hq,Hkv", REFERENCE_TEST_CASES + MORE_CASES)
@pytest.mark.parametrize("flavour", ["uniform", "peaked", "spread"])
def test_flash_prefill_matches_exact_attention_and_reference(orc, ref, n_new, cache_len, Hq, Hkv, flavour):
    from runtherder_b200 import kernels as K
    D = 128
    kw = {"uniform": dict(), "peaked": dict(q_mul=8.0), "spread": dict(q_mul=4.0, dist="normal", v_spread=2.0)}[flavour]
    q, kc, ks, vc, vs = make_case(n_new, cache_len, Hq, Hkv, D, seed=n_new * 7 + cache_len, **kw)
    scale = 1.0 / math.sqrt(D)
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    outs = {}
    try:
        # 16 or 32 query rows per warp (mma.sync); 128 rows per CTA in tensor memory (tcgen05) with 1, 2 or 4
        # threads sharing a row, and (3, the default) the accumulator-fragment form
        for tiles, parts in ((1, 0), (2, 0), (3, 1), (3, 2), (3, 3), (3, 4), (3, 5), (3, 6)):
            K.tune("prefill_tiles", tiles)
            K.tune("prefill_parts", parts)
            key = tiles if tiles < 3 else 10 * tiles + parts
            outs[key] = torch.full((n_new, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
            K.flash_prefill_bf16(outs[key], q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
    finally:
        K.tune("prefill_tiles", 0)
        K.tune("prefill_parts", 0)
    out = outs[1]
    out_naive, out_flash = torch.empty_like(out), torch.empty_like(out)
    ref.attention_causal_bf16(out_naive, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
    ref.flash_prefill_bf16(out_flash, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    exact_bits, exact = orc.attention_causal_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    check(outs[1], exact_bits, exact, "this library, 16 rows per warp")
    check(outs[2], exact_bits, exact, "this library, 32 rows per warp")
    for parts in (1, 2, 4):
        check(outs[30 + parts], exact_bits, exact, f"this library, tensor-memory form, {parts} thread(s) per row")
    check(outs[33], exact_bits, exact, "this library, tensor-memory form, accumulator-fragment reads")
    check(outs[35], exact_bits, exact, "this library, tensor-memory form, warps split by role")
    check(outs[36], exact_bits, exact, "this library, tensor-memory form, warps split by role, two row blocks per CTA")
    check(out_naive, exact_bits, exact, "reference naive kernel", significance=64)
    a, b = out_naive.float().flatten(), out.float().flatten()
    if flavour != "spread":
        assert float((a - b).abs().max()) <= 5e-2
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) >= 0.998
    # the reference's flash kernel rounds K*scale and V*scale to f16: it stays within its own test's bounds
    f = out_flash.float().flatten()
    assert float(torch.dot(a, f) / (a.norm() * f.norm())) >= 0.998


@pytest.mark.parametrize("parts", [0, 6, 5, 3, 2])
def test_zero_rows_extreme_value_scales_and_an_all_zero_value_cache(orc, parts):
    """Keys whose K or V row is all zero (scale 0), V rows of magnitude 1e-6 and 1e+4 side by side, a run of
    small ones: the V scale lives in the weight's exponent and in the denominators' multiplier, and both must
    stay exact; an all-zero value cache gives exact zeros, not NaN.  Default form, the role-split forms with
    two and one row block, and the single-role forms."""
    from runtherder_b200 import kernels as K
    n_new, cache_len, Hq, Hkv, D = 150, 90, 8, 2, 128
    g = torch.Generator(device="cuda").manual_seed(23)
    n = cache_len + n_new
    q = (torch.randn(n_new, Hq, D, device="cuda", generator=g) * 2.0).to(torch.bfloat16)
    k = torch.randn(n, Hkv, D, device="cuda", generator=g)
    v = torch.randn(n, Hkv, D, device="cuda", generator=g)
    k[5] = 0.0
    k[130] = 0.0
    v[7] = 0.0
    v[9] *= 1e-6
    v[11] *= 1e4
    v[100:120] *= 1e-3
    v[200] = 0.0
    at = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda"); vc = torch.empty_like(kc)
    ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda"); vs = torch.empty_like(ks)
    K.quantize_kv_fp8(kc, ks, k.to(torch.bfloat16), at, 1, n * Hkv, D)
    K.quantize_kv_fp8(vc, vs, v.to(torch.bfloat16), at, 1, n * Hkv, D)
    assert float(ks[5].abs().max()) == 0.0 and float(vs[7].abs().max()) == 0.0
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(D)
    exact_bits, exact = orc.attention_causal_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    try:
        K.tune("prefill_parts", parts)
        out = torch.full((n_new, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.flash_prefill_bf16(out, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
        torch.cuda.synchronize()
        check(out, exact_bits, exact, f"prefill_parts={parts}")
        vc.zero_(); vs.zero_()
        K.flash_prefill_bf16(out, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
        torch.cuda.synchronize()
        assert float(out.float().abs().max()) == 0.0
    finally:
        K.tune("prefill_parts", 0)


def test_prefill_then_decode_agree_on_the_last_token(orc):
    """The last token of a prefill is a decode step over the same cache: both entry points must land on the
    same exact value."""
    from runtherder_b200 import kernels as K
    n_new, cache_len, Hq, Hkv, D = 150, 40, 24, 8, 128
    q, kc, ks, vc, vs = make_case(n_new, cache_len, Hq, Hkv, D, seed=5, q_mul=3.0, dist="normal")
    scale = 1.0 / math.sqrt(D)
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    out = torch.empty(n_new, Hq, D, dtype=torch.bfloat16, device="cuda")
    K.flash_prefill_bf16(out, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
    last = torch.tensor([cache_len + n_new - 1], dtype=torch.int32, device="cuda")
    part = torch.empty(K.flash_split_scratch_floats(Hq, D, 8), dtype=torch.float32, device="cuda")
    dec = torch.empty(Hq, D, dtype=torch.bfloat16, device="cuda")
    K.flash_decode_split_bf16(dec, q[n_new - 1].contiguous(), kc, vc, ks, vs, part, 8, last, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    bits, exact = orc.attention_decode_fp8(to_np(q[n_new - 1].contiguous()), to_np(kc), to_np(vc), to_np(ks), to_np(vs),
                                           cache_len + n_new - 1, scale)
    check(out[n_new - 1], bits, exact, "prefill, last token")
    check(dec, bits, exact, "decode", significance=64)


def test_full_size_prefill_properties(orc):
    """The prefill configuration's full size (8192 tokens, 32/8 heads): (a) the tensor-memory form and the
    mma.sync form land within two ulp-at-row-max of each other everywhere, (b) sampled tokens match the exact
    value, (c) a chunked prefill of the tail (different row-to-CTA grouping, `*cache_len` > 0) reproduces the
    same rows of the whole prefill bit for bit."""
    from runtherder_b200 import kernels as K
    T, Hq, Hkv, D = 8192, 32, 8, 128
    q, kc, ks, vc, vs = make_case(T, 0, Hq, Hkv, D, seed=77, q_mul=3.0, dist="normal")
    scale = 1.0 / math.sqrt(D)
    zero = torch.zeros(1, dtype=torch.int32, device="cuda")
    out_tc = torch.empty(T, Hq, D, dtype=torch.bfloat16, device="cuda")
    out_mma = torch.empty_like(out_tc)
    K.flash_prefill_bf16(out_tc, q, kc, vc, ks, vs, T, zero, Hq, Hkv, D, scale)
    try:
        K.tune("prefill_tiles", 2)
        K.flash_prefill_bf16(out_mma, q, kc, vc, ks, vs, T, zero, Hq, Hkv, D, scale)
    finally:
        K.tune("prefill_tiles", 0)
    torch.cuda.synchronize()
    a, b = out_tc.float(), out_mma.float()
    assert bool(torch.isfinite(a).all())
    rowmax = b.abs().amax(dim=-1, keepdim=True)
    assert float(((a - b).abs() / rowmax).max()) <= 2 * ROWMAX_TOL
    for t0, n in ((0, 3), (62, 4), (4094, 4), (T - 4, 4)):
        bits, exact = orc.attention_causal_fp8(to_np(q[t0:t0 + n].contiguous()), to_np(kc[:t0 + n]), to_np(vc[:t0 + n]),
                                               to_np(ks[:t0 + n]), to_np(vs[:t0 + n]), t0, scale)
        check(out_tc[t0:t0 + n].contiguous(), bits, exact, f"tokens {t0}..{t0 + n - 1} of {T}")
    t0 = 4100                                   # not a multiple of the token tile: rows regroup
    cl = torch.tensor([t0], dtype=torch.int32, device="cuda")
    tail = torch.empty(T - t0, Hq, D, dtype=torch.bfloat16, device="cuda")
    K.flash_prefill_bf16(tail, q[t0:].contiguous(), kc, vc, ks, vs, T - t0, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    assert torch.equal(tail.view(torch.int16), out_tc[t0:].view(torch.int16))


def test_output_that_is_only_four_byte_aligned(orc):
    """The reference asks nothing of `out` beyond bf16 pairs; the tensor-memory form stores 16-byte pieces, so such
    a call takes the mma.sync form and must land on the same exact values."""
    from runtherder_b200 import kernels as K
    n_new, cache_len, Hq, Hkv, D = 70, 9, 8, 2, 128
    q, kc, ks, vc, vs = make_case(n_new, cache_len, Hq, Hkv, D, seed=21, q_mul=2.0, dist="normal")
    scale = 1.0 / math.sqrt(D)
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    backing = torch.zeros(n_new * Hq * D + 8, dtype=torch.bfloat16, device="cuda")
    out = backing[2:2 + n_new * Hq * D].view(n_new, Hq, D)
    assert out.data_ptr() % 16 == 4
    K.flash_prefill_bf16(out, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    bits, exact = orc.attention_causal_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    check(out.contiguous(), bits, exact, "four-byte aligned output")
    assert float(backing[:2].float().abs().max()) == 0.0 and float(backing[-6:].float().abs().max()) == 0.0


def test_cache_len_is_read_on_the_device_and_arguments_are_checked():
    from runtherder_b200 import _lib
    from runtherder_b200 import kernels as K
    n_new, Hq, Hkv, D = 40, 8, 2, 128
    q, kc, ks, vc, vs = make_case(n_new, 100, Hq, Hkv, D, seed=9)
    out_a = torch.empty(n_new, Hq, D, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty_like(out_a)
    cl = torch.tensor([100], dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        K.flash_prefill_bf16(out_a, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 0.1)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            K.flash_prefill_bf16(out_a, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 0.1)
    for depth in (0, 37, 100):
        cl.fill_(depth)
        graph.replay()
        K.flash_prefill_bf16(out_b, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 0.1)
        torch.cuda.synchronize()
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
        if depth != 100:
            cl.fill_(100)
            K.flash_prefill_bf16(out_b, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 0.1)
            torch.cuda.synchronize()
            assert not torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))

    def status(n_new=n_new, Hq=Hq, Hkv=Hkv, D=D, cache=cl.data_ptr()):
        return _lib.lib.rh_flash_prefill_bf16(out_a.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                                              vs.data_ptr(), n_new, cache, Hq, Hkv, D, 0.1, None)
    assert status() == 0
    assert status(n_new=0) == 1 and status(Hq=3) == 1 and status(cache=None) == 1     # RH_ERR_INVALID_ARG
    assert status(D=64) == 2                                                          # RH_ERR_UNSUPPORTED_DIM
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode", ["prefill", "decode"])
def test_layer_chain_with_attention_feeds_the_attention_output_through(orc, mode):
    """fused_layer_step(..., attention_partial=...) runs RoPE + KV append, then the attention over the cache it
    just wrote (flash prefill for T > 1, split-KV flash decode for T = 1, as src/attention/adaptive.cu:24-41
    dispatches), then quantises the attention output: the attention result must match the oracle on the
    rotated q and the cache contents, and the INT8 codes must be those of that result."""
    from dataclasses import replace
    from runtherder_b200 import kernels as K, layer_ops, synth
    from runtherder_b200.configs import C0
    if mode == "prefill":
        cfg, hist = C0, 0
    else:
        hist = 150
        cfg = replace(C0, tokens=1, start_pos=hist, max_seq=hist + 1)
    T = cfg.tokens
    ins = synth.make_inputs(cfg)
    outs = layer_ops.alloc_outputs(cfg, T, slots=cfg.cache_slots)
    outs["at_pos"].fill_(hist)
    ins["positions"] = torch.arange(hist, hist + T, dtype=torch.int32, device="cuda")
    if hist:
        g = torch.Generator(device="cuda").manual_seed(4)
        zero = torch.zeros(1, dtype=torch.int32, device="cuda")
        for codes, scales in ((outs["k_cache"], outs["k_scale"]), (outs["v_cache"], outs["v_scale"])):
            x = torch.randn(hist, cfg.kv_heads, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)
            K.quantize_kv_fp8(codes, scales, x, zero, 1, hist * cfg.kv_heads, cfg.head_dim)
    partial = torch.empty(K.flash_split_scratch_floats(cfg.q_heads, cfg.head_dim, layer_ops.ATTENTION_SPLITS),
                          dtype=torch.float32, device="cuda")
    launches = layer_ops.fused_layer_step(cfg, ins, outs, attention_partial=partial)
    torch.cuda.synchronize()
    assert launches == 5 + (2 if T == 1 else 1)
    scale = 1.0 / math.sqrt(cfg.head_dim)
    q_rot = to_np(ins["q"]).reshape(T, cfg.q_heads, cfg.head_dim)
    bits, exact = orc.attention_causal_fp8(q_rot, to_np(outs["k_cache"])[:hist + T], to_np(outs["v_cache"])[:hist + T],
                                           to_np(outs["k_scale"])[:hist + T], to_np(outs["v_scale"])[:hist + T], hist, scale)
    attn = ins["attn"].view(T, cfg.q_heads, cfg.head_dim)
    check(attn, bits, exact, f"attention inside the {mode} chain")
    oq, os_ = orc.quant_int8(to_np(ins["attn"]).reshape(T, cfg.q_dim))
    assert np.array_equal(to_np(outs["q_attn_out"]), oq) and np.array_equal(to_np(outs["s_attn_out"]), os_)
