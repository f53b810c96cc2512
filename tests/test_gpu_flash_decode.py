"""Split-KV flash decode over the FP8 cache (rh_flash_decode_split_bf16) against
  * the double-precision oracle of the reference's attention formula (oracle/rh_oracle.c),
  * the reference's own CUDA kernels built for sm_100a: its naive attention (the oracle of the reference's
    tests/kernels/test_flash_decode.cpp) and its flash_decode_split_bf16,
on the reference test's four shapes, the decode configuration (depth 8196, 24/8 heads) and edge cases.

Tolerance.  The reference documents that split orders "differ in the last bits, not in value"
(include/runtherder/kernels/flash_decode.cuh:45-46) and its test accepts max-abs 3e-2 / cosine 0.999.  The bar
here is tighter: every element within ONE bf16 ulp of the correctly rounded exact value wherever the element is
not a cancellation residue (|exact| >= row max / 64), and within 1.5 * 2^-7 of the row maximum everywhere —
the same bar the reference's own two kernels meet on these inputs."""
import math

import numpy as np
import pytest
import torch

from gpu_util import ref_cuda_or_skip, to_np
from oracle_lib import Oracle

pytestmark = pytest.mark.gpu

ULP_TOL = 1
ROWMAX_TOL = 1.5 * 2.0 ** -7


@pytest.fixture(scope="module")
def orc():
    return Oracle()


@pytest.fixture(scope="module")
def ref():
    try:
        return ref_cuda_or_skip()
    except RuntimeError as exc:
        pytest.skip(str(exc))


def ordered(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)


def make_case(cache_len, Hq, Hkv, D, seed, q_mul=1.0, dist="uniform", v_spread=0.0):
    """Seeded q/K/V; K and V go through the library's FP8 cache writer (bit-identical to the reference's)."""
    from runtherder_b200 import kernels as K
    g = torch.Generator(device="cuda").manual_seed(seed)
    n = cache_len + 1
    if dist == "uniform":                      # the reference test's distribution: U(-1, 1)
        q = (torch.rand(Hq, D, device="cuda", generator=g) * 2 - 1) * q_mul
        k = torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1
        v = torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1
    else:
        q = torch.randn(Hq, D, device="cuda", generator=g) * q_mul
        k = torch.randn(n, Hkv, D, device="cuda", generator=g)
        v = torch.randn(n, Hkv, D, device="cuda", generator=g)
    if v_spread:                                # per-row magnitudes over e^(+-2*spread): scales differ by orders
        v = v * torch.exp(torch.randn(n, Hkv, 1, device="cuda", generator=g) * v_spread)
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    at = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda")
    vc = torch.empty_like(kc)
    ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda")
    vs = torch.empty_like(ks)
    K.quantize_kv_fp8(kc, ks, k, at, 1, n * Hkv, D)
    K.quantize_kv_fp8(vc, vs, v, at, 1, n * Hkv, D)
    return q, kc, ks, vc, vs


def run_ours(q, kc, ks, vc, vs, cache_len, splits, scale):
    from runtherder_b200 import kernels as K
    Hq, D = q.shape
    Hkv = kc.shape[1]
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    part = torch.full((K.flash_split_scratch_floats(Hq, D, splits),), float("nan"), dtype=torch.float32, device="cuda")
    out = torch.empty(Hq, D, dtype=torch.bfloat16, device="cuda")
    K.flash_decode_split_bf16(out, q, kc, vc, ks, vs, part, splits, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    return out


def check_against_exact(out: torch.Tensor, exact_bits: np.ndarray, exact_f32: np.ndarray, what: str):
    got_bits = to_np(out)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all(), what
    rowmax = np.abs(exact_f32).max(axis=1, keepdims=True)
    err = np.abs(got - exact_f32)
    assert (err <= ROWMAX_TOL * rowmax + 1e-30).all(), (what, float((err / rowmax).max()))
    significant = np.abs(exact_f32) >= rowmax / 64
    ulp = np.abs(ordered(got_bits) - ordered(exact_bits))
    assert ulp[significant].max(initial=0) <= ULP_TOL, (what, int(ulp[significant].max()))


REFERENCE_TEST_CASES = [(300, 32, 8, 128, 4), (0, 32, 8, 128, 1), (2, 8, 2, 64, 8), (1000, 32, 8, 128, 8)]
MORE_CASES = [
    (8195, 24, 8, 128, 32),    # the decode configuration: Llama-3.2-3B at depth 8196, the reference's 32 splits
    (777, 28, 4, 128, 32),     # Qwen2-7B grouping: 7 query heads per kv head
    (500, 16, 1, 64, 5),       # 16 query heads on one kv head: two row chunks per split
    (333, 8, 8, 32, 3),        # no grouping, head_dim 32
    (600, 8, 2, 256, 7),       # head_dim 256 (single-buffered path)
    (15, 4, 4, 128, 2), (16, 4, 2, 128, 1), (17, 4, 2, 128, 3),   # around the 16-key tile
    (40, 6, 2, 64, 64),        # more splits than tiles
]


@pytest.mark.parametrize("cache_len,Hq,Hkv,D,splits", REFERENCE_TEST_CASES + MORE_CASES)
@pytest.mark.parametrize("flavour", ["uniform", "peaked", "spread"])
def test_flash_decode_matches_exact_attention_and_reference(orc, ref, cache_len, Hq, Hkv, D, splits, flavour):
    kw = {"uniform": dict(), "peaked": dict(q_mul=8.0), "spread": dict(q_mul=4.0, dist="normal", v_spread=2.0)}[flavour]
    q, kc, ks, vc, vs = make_case(cache_len, Hq, Hkv, D, seed=cache_len + 7 * splits, **kw)
    scale = 1.0 / math.sqrt(D)
    out = run_ours(q, kc, ks, vc, vs, cache_len, splits, scale)
    exact_bits, exact = orc.attention_decode_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    check_against_exact(out, exact_bits, exact, "this library")

    # the reference's kernels meet the same bar against the same oracle: that pins the oracle to them
    from runtherder_b200 import kernels as K
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    out_naive, out_split = torch.empty_like(out), torch.empty_like(out)
    part = torch.empty(K.flash_split_scratch_floats(Hq, D, splits), dtype=torch.float32, device="cuda")
    ref.attention_causal_bf16(out_naive, q, kc, vc, ks, vs, 1, cl, Hq, Hkv, D, scale)
    ref.flash_decode_split_bf16(out_split, q, kc, vc, ks, vs, part, splits, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    check_against_exact(out_naive, exact_bits, exact, "reference naive kernel")
    check_against_exact(out_split, exact_bits, exact, "reference split kernel")

    # and the reference test's own acceptance (tests/kernels/test_flash_decode.cpp:97-98,145-149); its absolute
    # bound is meant for its own value range, |v| <= 1
    a, b = out_naive.float().flatten(), out.float().flatten()
    if flavour != "spread":
        assert float((a - b).abs().max()) <= 3e-2
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) >= 0.999


def test_any_split_count_gives_the_same_attention(orc):
    cache_len, Hq, Hkv, D = 1234, 12, 4, 128
    q, kc, ks, vc, vs = make_case(cache_len, Hq, Hkv, D, seed=3, q_mul=3.0, dist="normal")
    scale = 0.09
    exact_bits, exact = orc.attention_decode_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    for splits in (1, 2, 3, 7, 32, 77, 78, 200, 2000):
        check_against_exact(run_ours(q, kc, ks, vc, vs, cache_len, splits, scale), exact_bits, exact, f"splits={splits}")


def test_extreme_scales_zero_rows_and_large_queries(orc):
    """Rows whose scale is 0 (all-zero K or V row), V rows 1e-6 and 1e+4 in magnitude side by side, q of
    magnitude 1e3 (one-hot softmax) and 1e-20 (flat softmax): the exponent-domain handling of the V scale
    and the power-of-two scaling of q must stay exact.  (Logits far beyond that, |q| ~ 3e4, leave the
    one-ulp bar for any fp32 evaluation; the tensor-core accumulation reaches 0.7 % of the row maximum
    there, the reference's FMA chains 0.25 %.)"""
    from runtherder_b200 import kernels as K
    cache_len, Hq, Hkv, D = 200, 8, 2, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    n = cache_len + 1
    k = torch.randn(n, Hkv, D, device="cuda", generator=g)
    v = torch.randn(n, Hkv, D, device="cuda", generator=g)
    k[5] = 0.0
    v[7] = 0.0
    v[9] *= 1e-6
    v[11] *= 1e4
    v[100:120] *= 1e-3
    at = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda"); vc = torch.empty_like(kc)
    ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda"); vs = torch.empty_like(ks)
    K.quantize_kv_fp8(kc, ks, k.to(torch.bfloat16), at, 1, n * Hkv, D)
    K.quantize_kv_fp8(vc, vs, v.to(torch.bfloat16), at, 1, n * Hkv, D)
    assert float(ks[5].abs().max()) == 0.0 and float(vs[7].abs().max()) == 0.0
    for q_mul in (1.0, 30.0, 1e3, 1e-20):       # logits up to ~2e3 in magnitude
        q = (torch.randn(Hq, D, device="cuda", generator=g) * q_mul).to(torch.bfloat16)
        exact_bits, exact = orc.attention_decode_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, 0.1)
        check_against_exact(run_ours(q, kc, ks, vc, vs, cache_len, 6, 0.1), exact_bits, exact, f"q_mul={q_mul}")
    # an all-zero value cache gives exact zeros, not NaN
    vc.zero_(); vs.zero_()
    out = run_ours(q, kc, ks, vc, vs, cache_len, 6, 0.1)
    assert float(out.float().abs().max()) == 0.0


def test_cache_len_is_read_on_the_device_at_replay(orc):
    """The decode loop replays one graph with a growing history (src/engine/generator.cu:46-68): the kernel
    must pick up *cache_len at execution time, and run after the cache append of the same step."""
    from runtherder_b200 import kernels as K
    Hq, Hkv, D, splits, depth = 24, 8, 128, 32, 700
    q, kc, ks, vc, vs = make_case(depth - 1, Hq, Hkv, D, seed=21, q_mul=2.0, dist="normal")
    g = torch.Generator(device="cuda").manual_seed(22)
    k_new = torch.randn(1, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v_new = torch.randn(1, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    kc0, ks0, vc0, vs0 = kc.clone(), ks.clone(), vc.clone(), vs.clone()
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    part = torch.empty(K.flash_split_scratch_floats(Hq, D, splits), dtype=torch.float32, device="cuda")
    out = torch.empty(Hq, D, dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / math.sqrt(D)

    def step():
        K.quantize_kv_fp8(kc, ks, k_new, pos, Hkv, Hkv, D)          # append at slot *pos ...
        K.quantize_kv_fp8(vc, vs, v_new, pos, Hkv, Hkv, D)
        K.flash_decode_split_bf16(out, q, kc, vc, ks, vs, part, splits, pos, Hq, Hkv, D, scale)   # ... attend 0..*pos

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        pos.fill_(3)
        step()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step()
    for p in (0, 15, 16, 333, depth - 1):
        for dst, src in ((kc, kc0), (ks, ks0), (vc, vc0), (vs, vs0)):
            dst.copy_(src)
        pos.fill_(p)
        graph.replay()
        torch.cuda.synchronize()
        exact_bits, exact = orc.attention_decode_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), p, scale)
        check_against_exact(out, exact_bits, exact, f"replay at position {p}")
        assert not torch.equal(kc[p], kc0[p])           # the step's own append is part of the history


@pytest.mark.parametrize("cache_len,Hq,Hkv,splits", [(300, 8, 2, 4), (1000, 4, 4, 8), (0, 2, 1, 3), (77, 6, 2, 32)])
def test_flash_decode_head_dim_512(orc, ref, cache_len, Hq, Hkv, splits):
    """head_dim 512, which the reference's split kernel accepts (src/kernels/flash_decode.cu:313-314) and its
    naive kernel does not (attention.cu:116, at most 256): this library and the reference's split kernel are
    both held to the exact attention."""
    D = 512
    q, kc, ks, vc, vs = make_case(cache_len, Hq, Hkv, D, seed=cache_len + 3 * splits)
    scale = 1.0 / math.sqrt(D)
    out = run_ours(q, kc, ks, vc, vs, cache_len, splits, scale)
    exact_bits, exact = orc.attention_decode_fp8(to_np(q), to_np(kc), to_np(vc), to_np(ks), to_np(vs), cache_len, scale)
    check_against_exact(out, exact_bits, exact, "this library, head_dim 512")
    from runtherder_b200 import kernels as K
    cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
    out_split = torch.empty_like(out)
    part = torch.empty(K.flash_split_scratch_floats(Hq, D, splits), dtype=torch.float32, device="cuda")
    ref.flash_decode_split_bf16(out_split, q, kc, vc, ks, vs, part, splits, cl, Hq, Hkv, D, scale)
    torch.cuda.synchronize()
    check_against_exact(out_split, exact_bits, exact, "reference split kernel, head_dim 512")


def test_argument_checks():
    from runtherder_b200 import _lib
    from runtherder_b200 import kernels as K
    assert K.flash_split_scratch_floats(24, 128, 32) == 24 * 32 * 2 + 24 * 32 * 128      # flash_decode.cuh:16-25
    assert K.flash_split_scratch_floats(0, 128, 32) == 0
    q, kc, ks, vc, vs = make_case(10, 4, 2, 64, seed=1)
    cl = torch.tensor([10], dtype=torch.int32, device="cuda")
    part = torch.empty(K.flash_split_scratch_floats(4, 512, 4), dtype=torch.float32, device="cuda")
    out = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")

    def status(**over):
        a = dict(num_splits=4, Hq=4, Hkv=2, D=64)
        a.update(over)
        return _lib.lib.rh_flash_decode_split_bf16(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                                                   vs.data_ptr(), part.data_ptr(), a["num_splits"], cl.data_ptr(), a["Hq"],
                                                   a["Hkv"], a["D"], 0.125, None)
    assert status() == 0
    assert status(num_splits=0) == 1                     # RH_ERR_INVALID_ARG
    assert status(Hq=3) == 1                             # not divisible by the kv heads
    assert status(D=48) == 2 and status(D=1024) == 2     # RH_ERR_UNSUPPORTED_DIM (nothing is launched)
    assert _lib.lib.rh_flash_decode_split_bf16(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                                               vs.data_ptr(), part.data_ptr(), 4, None, 4, 2, 64, 0.125, None) == 1
    torch.cuda.synchronize()
