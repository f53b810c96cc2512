"""CUDA kernels (through the C ABI) against the CPU oracle on the same seeded inputs.

Bit-exact: INT8 codes and scales, FP8 bytes and scales, gathered rows, h_out, frequency tables.
bf16 outputs of the norm, RoPE and SwiGLU are held to 1 bf16 ulp where the oracle's double-precision
arithmetic can only differ by rounding, and to the reference tests' own tolerance (max-abs 5e-2,
cosine >= 0.9999) otherwise — the device uses rsqrtf/__expf/__sincosf like the reference kernels do.
"""
import numpy as np
import pytest
import torch

from oracle_lib import Oracle, bf16_to_f32, bf16_ulp_diff
from refgen import f32_to_bf16, make_bf16_random

pytestmark = pytest.mark.gpu

ORC = Oracle()
ABS_TOL, COS_FLOOR = 5e-2, 0.9999   # tests/kernels/test_rmsnorm.cpp:129-130 and its siblings


def _k():
    from runtherder_b200 import kernels
    return kernels


def _gpu():
    from gpu_util import to_dev, to_np
    return to_dev, to_np


def check_close(got_u16, want_u16, max_ulp=1, frac_off=2e-3):
    """Reference-test tolerance always; additionally at most `max_ulp` bf16 ulp on all but a tiny fraction."""
    a, b = bf16_to_f32(got_u16).astype(np.float64).ravel(), bf16_to_f32(want_u16).astype(np.float64).ravel()
    assert np.abs(a - b).max() <= ABS_TOL
    denom = np.sqrt((a * a).sum()) * np.sqrt((b * b).sum())
    if denom > 0:
        assert (a * b).sum() / denom >= COS_FLOOR
    ulp = bf16_ulp_diff(got_u16.ravel(), want_u16.ravel())
    assert (ulp > max_ulp).mean() <= frac_off, f"{(ulp > max_ulp).sum()} of {ulp.size} beyond {max_ulp} ulp"


@pytest.mark.parametrize("T,H", [(1, 128), (4, 2560), (2, 16384), (32, 2560), (35, 3072), (3, 8), (5, 4096), (2, 264)])
def test_rmsnorm_and_add(T, H):
    K = _k(); to_dev, to_np = _gpu()
    x, r = make_bf16_random(T * H, 1.0, 0xFEEDFACE).reshape(T, H), make_bf16_random(T * H, 1.0, 0xDEADBEEF).reshape(T, H)
    g = make_bf16_random(H, 0.5, 0xCAFEBABE)
    xd, rd, gd = to_dev(x), to_dev(r), to_dev(g)
    y = torch.empty_like(xd)
    K.rmsnorm_bf16_forward(y, xd, gd, T, H, 1e-5)
    check_close(to_np(y), ORC.rmsnorm(x, g, 1e-5))
    h = torch.empty_like(xd)
    K.rmsnorm_add_bf16_forward(y, h, xd, rd, gd, T, H, 1e-5)
    oy, oh = ORC.rmsnorm_add(x, r, g, 1e-5)
    assert np.array_equal(to_np(h), oh)              # bf16(x + r): exact on both sides
    check_close(to_np(y), oy)


@pytest.mark.parametrize("T,K_", [(1, 8), (35, 3072), (7, 128), (16, 8192), (3, 16384), (9, 1000), (4, 264)])
def test_quantize_per_token_int8(T, K_):
    K = _k(); to_dev, to_np = _gpu()
    x = make_bf16_random(T * K_, 4.0, 99 + T).reshape(T, K_)
    if T > 2:
        x[1] = 0                                     # zero row: scale 0, codes 0
    q = torch.empty(T, K_, dtype=torch.int8, device="cuda")
    s = torch.empty(T, dtype=torch.float32, device="cuda")
    K.quantize_per_token_int8(q, s, to_dev(x), T, K_)
    oq, os_ = ORC.quant_int8(x)
    assert np.array_equal(to_np(q), oq)
    assert np.array_equal(to_np(s).view(np.uint32), os_.view(np.uint32))


def test_quantize_int8_nonfinite_and_tiny_rows():
    """Rows holding NaN / Inf / subnormal-only values take the exact conversion path and still match."""
    K = _k(); to_dev, to_np = _gpu()
    T, K_ = 6, 3072
    xf = np.random.default_rng(5).normal(size=(T, K_)).astype(np.float32)
    xf[0, 17] = np.nan
    xf[1, 100] = np.inf
    xf[2, 5] = -np.inf; xf[2, 6] = np.nan
    xf[3] *= 1e-39                                    # subnormal amax: 127/amax overflows to inf
    xf[4] = 0; xf[4, 9] = 9.2e-41
    x = f32_to_bf16(xf)
    q = torch.empty(T, K_, dtype=torch.int8, device="cuda")
    s = torch.empty(T, dtype=torch.float32, device="cuda")
    K.quantize_per_token_int8(q, s, to_dev(x), T, K_)
    oq, os_ = ORC.quant_int8(x)
    assert np.array_equal(to_np(q), oq)
    assert np.array_equal(to_np(s).view(np.uint32), os_.view(np.uint32))


@pytest.mark.parametrize("R,D,at,rpp", [(24, 128, 0, 1), (8, 256, 0, 1), (512, 128, 0, 1), (2, 128, 0, 1),
                                        (24, 128, 5, 8), (8, 128, 8195, 8), (6, 64, 3, 2), (4, 2048, 2, 4),
                                        (5, 8, 1, 1)])
def test_quantize_kv_fp8(R, D, at, rpp):
    K = _k(); to_dev, to_np = _gpu()
    x = make_bf16_random(R * D, 1.0, 0xC0FFEE).reshape(R, D)
    if R == 2:
        x[:] = 0                                     # test_quantization.cpp:138-170
    slots = at * rpp + R + 3
    q = torch.zeros(slots, D, dtype=torch.uint8, device="cuda")
    s = torch.zeros(slots, dtype=torch.float32, device="cuda")
    at_dev = torch.tensor([at], dtype=torch.int32, device="cuda")
    K.quantize_kv_fp8(q, s, to_dev(x), at_dev, rpp, R, D)
    oq, os_ = ORC.quant_kv(x, at, rpp, slots)
    assert np.array_equal(to_np(q), oq)              # includes: nothing outside the target rows is touched
    assert np.array_equal(to_np(s).view(np.uint32), os_.view(np.uint32))
    deq = K.dequantize_kv_fp8(q, s)                  # read side: float(q) * scale
    lut = np.array([ORC.lib.orc_e4m3_to_f32(b) for b in range(256)], np.float32)
    want = lut[oq] * os_[:, None]
    assert np.array_equal(to_np(deq), want.astype(np.float32))


@pytest.mark.parametrize("n", [128, 9728, 8 * 9728, 32 * 9728, 8, 35 * 8192])
def test_swiglu(n):
    K = _k(); to_dev, to_np = _gpu()
    g, u = make_bf16_random(n, 2.0, 0xC0FFEE), make_bf16_random(n, 2.0, 0xBADBEEF)
    y = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    K.swiglu_bf16_forward(y, to_dev(g), to_dev(u), n)
    check_close(to_np(y), ORC.swiglu(g, u))
    gd = to_dev(g)                                   # aliasing y == gate (test_activation.cpp:125-150)
    K.swiglu_bf16_forward(gd, gd, to_dev(u), n)
    assert np.array_equal(to_np(gd), to_np(y))
    ud = to_dev(u)                                   # aliasing y == up
    K.swiglu_bf16_forward(ud, to_dev(g), ud, n)
    assert np.array_equal(to_np(ud), to_np(y))


@pytest.mark.parametrize("T,Hq,Hkv,D,theta,pos", [(1, 4, 1, 64, 1.0e4, 0), (8, 32, 8, 128, 1.0e6, 0),
                                                   (1, 32, 8, 128, 1.0e6, 1024), (2, 8, 2, 256, 1.0e6, 0),
                                                   (32, 32, 8, 128, 1.0e6, 0), (3, 5, 3, 96, 1.0e4, 7),
                                                   (35, 24, 8, 128, 5.0e5, 0), (2, 3, 1, 16, 1.0e4, 2)])
def test_rope(T, Hq, Hkv, D, theta, pos):
    K = _k(); to_dev, to_np = _gpu()
    q = make_bf16_random(T * Hq * D, 1.0, 0xC0FFEE).reshape(T, Hq, D)
    k = make_bf16_random(T * Hkv * D, 1.0, 0xBADBEEF).reshape(T, Hkv, D)
    inv = ORC.inv_freq_plain(D, theta)
    positions = np.arange(pos, pos + T, dtype=np.int32)
    qd, kd = to_dev(q), to_dev(k)
    K.rope_bf16(qd, kd, to_dev(positions), to_dev(inv), T, Hq, Hkv, D)
    check_close(to_np(qd), ORC.rope_theta(q, pos, theta), max_ulp=1, frac_off=2e-2)
    check_close(to_np(kd), ORC.rope_theta(k, pos, theta), max_ulp=1, frac_off=2e-2)
    check_close(to_np(qd), ORC.rope_table(q, positions, inv), max_ulp=1, frac_off=2e-2)


def test_embedding_gather():
    K = _k(); to_dev, to_np = _gpu()
    rng = np.random.default_rng(1)
    for V, H, T in [(1000, 3072, 35), (517, 8, 3), (128256, 64, 511), (300, 4096, 1)]:
        table = rng.integers(0, 65536, (V, H), dtype=np.uint16)
        ids = rng.integers(0, V, T, dtype=np.int32)
        out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        K.embedding_lookup_bf16_forward(out, to_dev(table), to_dev(ids), T, H)
        assert np.array_equal(to_np(out), table[ids])


@pytest.mark.parametrize("n,q_dim,kv_dim", [(3, 64, 16), (1, 1536, 256), (511, 2048, 256), (35, 3072, 1024), (2, 8, 8)])
def test_qkv_bias_add(n, q_dim, kv_dim):
    """Bit-identical to bf16(float(x) + float(b)) (tests/kernels/test_bias.cpp:46-57), shapes and seeds of that test."""
    K = _k(); to_dev, to_np = _gpu()
    q, k, v = (make_bf16_random(n * d, 4.0, s).reshape(n, d) for d, s in ((q_dim, 0x1111), (kv_dim, 0x2222), (kv_dim, 0x3333)))
    qb, kb, vb = (make_bf16_random(d, 2.0, s) for d, s in ((q_dim, 0x4444), (kv_dim, 0x5555), (kv_dim, 0x6666)))
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    K.qkv_bias_add_bf16_forward(qd, kd, vd, to_dev(qb), to_dev(kb), to_dev(vb), n, q_dim, kv_dim)
    assert np.array_equal(to_np(qd), ORC.add_rows(q, qb))
    assert np.array_equal(to_np(kd), ORC.add_rows(k, kb))
    assert np.array_equal(to_np(vd), ORC.add_rows(v, vb))


@pytest.mark.parametrize("T,Hq,Hkv,D", [(35, 28, 4, 128), (511, 28, 4, 128), (7, 6, 2, 128), (19, 12, 2, 64), (1, 28, 4, 128)])
def test_bias_fused_into_rope_kv_equals_the_two_step_sequence(T, Hq, Hkv, D):
    """rh_bias_rope_kv_fp8 (Qwen2: projection biases + RoPE + FP8 KV append in one launch) against the sequence
    it replaces — qkv_bias_add_bf16_forward, then RoPE + append — on the same inputs: rotated q, rotated k, both
    caches and their scales bit-identical; v_in untouched.  Qwen2-7B heads (28/4, the aligned kernel), head
    counts that are not a multiple of the heads per warp (the generic kernel), head_dim 64, one token."""
    K = _k(); to_dev, to_np = _gpu()
    from runtherder_b200 import rope_tables
    g = torch.Generator(device="cuda").manual_seed(T * 31 + Hq)
    q = (torch.randn(T, Hq, D, device="cuda", generator=g) * 2).to(torch.bfloat16)
    k = (torch.randn(T, Hkv, D, device="cuda", generator=g) * 2).to(torch.bfloat16)
    v = (torch.randn(T, Hkv, D, device="cuda", generator=g) * 2).to(torch.bfloat16)
    qb, kb, vb = ((torch.randn(h * D, device="cuda", generator=g)).to(torch.bfloat16) for h in (Hq, Hkv, Hkv))
    start = 40
    positions = torch.arange(start, start + T, dtype=torch.int32, device="cuda")
    inv = torch.from_numpy(rope_tables.rope_inv_freq_plain(D, 1.0e6)).cuda()
    at = torch.tensor([start], dtype=torch.int32, device="cuda")
    slots = start + T + 2

    def caches():
        return (torch.zeros(slots, Hkv, D, dtype=torch.uint8, device="cuda"), torch.zeros(slots, Hkv, dtype=torch.float32, device="cuda"),
                torch.zeros(slots, Hkv, D, dtype=torch.uint8, device="cuda"), torch.zeros(slots, Hkv, dtype=torch.float32, device="cuda"))

    # two steps
    q1, k1, v1 = q.clone(), k.clone(), v.clone()
    kc1, ks1, vc1, vs1 = caches()
    K.qkv_bias_add_bf16_forward(q1, k1, v1, qb, kb, vb, T, Hq * D, Hkv * D)
    K.rope_kv_fp8(q1, k1, k1, v1, None, None, 1e-6, positions, inv, kc1, ks1, vc1, vs1, at, T, Hq, Hkv, D)
    # fused
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    kc2, ks2, vc2, vs2 = caches()
    K.bias_rope_kv_fp8(q2, k2, k2, v2, qb, kb, vb, positions, inv, kc2, ks2, vc2, vs2, at, T, Hq, Hkv, D)
    torch.cuda.synchronize()
    for a, b in ((q1, q2), (k1, k2), (kc1, kc2), (ks1, ks2), (vc1, vc2), (vs1, vs2)):
        assert np.array_equal(to_np(a), to_np(b))
    assert np.array_equal(to_np(v2), to_np(v))                      # read only
    assert np.array_equal(to_np(v1), ORC.add_rows(to_np(v).reshape(T, Hkv * D), to_np(vb)).reshape(T, Hkv, D))
    assert bool((ks2[start:start + T] > 0).all()) and bool((ks2[:start] == 0).all())


def test_dequantize_w8a8():
    K = _k(); to_dev, to_np = _gpu()
    rng = np.random.default_rng(2)
    for m, n in [(5, 12), (35, 3072), (3, 7), (16, 1026)]:
        acc = rng.integers(-300000, 300000, (m, n), dtype=np.int32)
        xs = rng.uniform(0.001, 0.1, m).astype(np.float32)
        ws = f32_to_bf16(rng.uniform(0.001, 0.05, n).astype(np.float32))
        y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        K.dequantize_w8a8(y, to_dev(acc), to_dev(xs), to_dev(ws), m, n)
        assert np.array_equal(to_np(y), ORC.dequant_w8a8(acc, xs, ws))


@pytest.mark.parametrize("T,H,with_res,with_y", [(35, 3072, True, True), (35, 3072, True, False), (4, 4096, False, True),
                                                 (3, 128, True, True), (2, 16384, True, False), (6, 264, False, False)])
def test_fused_norm_quant_is_self_consistent(T, H, with_res, with_y):
    """The fused kernel's codes are the oracle's quantisation of the fused kernel's own bf16 output, and
    that output equals the unfused kernel's — so any 1-ulp difference to the double-precision oracle is
    confined to the norm, never introduced by the fusion."""
    K = _k(); to_dev, to_np = _gpu()
    x, r = make_bf16_random(T * H, 1.0, 21).reshape(T, H), make_bf16_random(T * H, 1.0, 22).reshape(T, H)
    xf = bf16_to_f32(x); xf[:, ::197] *= 20.0; x = f32_to_bf16(xf)     # outlier channels
    g = make_bf16_random(H, 0.5, 23)
    xd, rd, gd = to_dev(x), to_dev(r), to_dev(g)
    q = torch.empty(T, H, dtype=torch.int8, device="cuda"); s = torch.empty(T, dtype=torch.float32, device="cuda")
    h = torch.empty_like(xd); y = torch.empty_like(xd) if with_y else None
    K.rmsnorm_add_quant_int8(q, s, h if with_res else None, y, xd, rd if with_res else None, gd, T, H, 1e-5)
    y_ref, h_ref = torch.empty_like(xd), torch.empty_like(xd)
    if with_res:
        K.rmsnorm_add_bf16_forward(y_ref, h_ref, xd, rd, gd, T, H, 1e-5)
        assert np.array_equal(to_np(h), to_np(h_ref))
    else:
        K.rmsnorm_bf16_forward(y_ref, xd, gd, T, H, 1e-5)
    if with_y:
        assert np.array_equal(to_np(y), to_np(y_ref))
    oq, os_ = ORC.quant_int8(to_np(y_ref))
    assert np.array_equal(to_np(q), oq)
    assert np.array_equal(to_np(s).view(np.uint32), os_.view(np.uint32))


@pytest.mark.parametrize("T,I,with_y", [(35, 8192, True), (35, 8192, False), (3, 14336, False), (5, 12288, True),
                                        (2, 128, True), (4, 4096, False), (2, 16384, False), (3, 9728, True)])
def test_fused_swiglu_quant_is_self_consistent(T, I, with_y):
    K = _k(); to_dev, to_np = _gpu()
    g, u = make_bf16_random(T * I, 3.0, 31).reshape(T, I), make_bf16_random(T * I, 3.0, 32).reshape(T, I)
    gd, ud = to_dev(g), to_dev(u)
    q = torch.empty(T, I, dtype=torch.int8, device="cuda"); s = torch.empty(T, dtype=torch.float32, device="cuda")
    y = torch.empty_like(gd) if with_y else None
    K.swiglu_quant_int8(q, s, y, gd, ud, T, I)
    y_ref = torch.empty_like(gd)
    K.swiglu_bf16_forward(y_ref, gd, ud, T * I)
    if with_y:
        assert np.array_equal(to_np(y), to_np(y_ref))
    oq, os_ = ORC.quant_int8(to_np(y_ref))
    assert np.array_equal(to_np(q), oq)
    assert np.array_equal(to_np(s).view(np.uint32), os_.view(np.uint32))
    check_close(to_np(y_ref), ORC.swiglu(g, u))


@pytest.mark.parametrize("T,Hq,Hkv,D,norm,at", [(35, 24, 8, 128, False, 0), (8, 32, 8, 128, True, 0),
                                                 (1, 24, 8, 128, False, 8195), (5, 6, 2, 64, True, 3),
                                                 (3, 8, 2, 256, False, 1), (4, 5, 3, 128, True, 2),
                                                 (2, 3, 1, 32, False, 0)])
def test_fused_rope_kv_is_self_consistent(T, Hq, Hkv, D, norm, at):
    """Fused [QK-norm +] RoPE + KV append == the unfused kernels chained (bit for bit), and the cache
    bytes are the oracle's FP8 quantisation of the rotated bf16 K the fused kernel itself wrote."""
    K = _k(); to_dev, to_np = _gpu()
    q = make_bf16_random(T * Hq * D, 1.0, 41).reshape(T, Hq, D)
    k = make_bf16_random(T * Hkv * D, 1.0, 42).reshape(T, Hkv, D)
    v = make_bf16_random(T * Hkv * D, 1.0, 43).reshape(T, Hkv, D)
    v[0, 0] = 0                                       # a zero head row: scale 0, bytes 0
    qn, kn = make_bf16_random(D, 0.5, 44), make_bf16_random(D, 0.5, 45)
    qn = f32_to_bf16(bf16_to_f32(qn) + 1.0); kn = f32_to_bf16(bf16_to_f32(kn) + 1.0)
    inv = ORC.inv_freq_llama3(D, 500000.0, 32.0, 1.0, 4.0, 8192)
    positions = np.arange(at, at + T, dtype=np.int32)
    slots = at + T + 2
    at_dev = torch.tensor([at], dtype=torch.int32, device="cuda")
    pd, fd = to_dev(positions), to_dev(inv)

    def caches():
        return (torch.zeros(slots, Hkv, D, dtype=torch.uint8, device="cuda"), torch.zeros(slots, Hkv, dtype=torch.float32, device="cuda"),
                torch.zeros(slots, Hkv, D, dtype=torch.uint8, device="cuda"), torch.zeros(slots, Hkv, dtype=torch.float32, device="cuda"))

    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    k_rot = torch.empty_like(kd)
    kc, ks, vc, vs = caches()
    K.rope_kv_fp8(qd, k_rot, kd, vd, to_dev(qn) if norm else None, to_dev(kn) if norm else None, 1e-6, pd, fd,
                  kc, ks, vc, vs, at_dev, T, Hq, Hkv, D)
    # unfused chain with this library's drop-in kernels
    q2, k2 = to_dev(q), to_dev(k)
    if norm:
        K.rmsnorm_bf16_forward(q2, q2, to_dev(qn), T * Hq, D, 1e-6)
        K.rmsnorm_bf16_forward(k2, k2, to_dev(kn), T * Hkv, D, 1e-6)
    K.rope_bf16(q2, k2, pd, fd, T, Hq, Hkv, D)
    kc2, ks2, vc2, vs2 = caches()
    K.quantize_kv_fp8(kc2, ks2, k2, at_dev, Hkv, T * Hkv, D)
    K.quantize_kv_fp8(vc2, vs2, vd, at_dev, Hkv, T * Hkv, D)
    for a, b in [(qd, q2), (k_rot, k2), (kc, kc2), (ks, ks2), (vc, vc2), (vs, vs2)]:
        assert np.array_equal(to_np(a).view(np.uint8), to_np(b).view(np.uint8))
    # cache bytes vs the oracle, from the kernel's own rotated K and the untouched V
    oq, os_ = ORC.quant_kv(to_np(k_rot).reshape(T * Hkv, D), at, Hkv, slots * Hkv)
    assert np.array_equal(to_np(kc).reshape(-1, D), oq) and np.array_equal(to_np(ks).ravel().view(np.uint32), os_.view(np.uint32))
    oq, os_ = ORC.quant_kv(v.reshape(T * Hkv, D), at, Hkv, slots * Hkv)
    assert np.array_equal(to_np(vc).reshape(-1, D), oq) and np.array_equal(to_np(vs).ravel().view(np.uint32), os_.view(np.uint32))
    # and the whole chain against the oracle chain within the reference tests' tolerance
    oqn = ORC.rmsnorm(q.reshape(-1, D), qn, 1e-6).reshape(q.shape) if norm else q
    okn = ORC.rmsnorm(k.reshape(-1, D), kn, 1e-6).reshape(k.shape) if norm else k
    check_close(to_np(qd), ORC.rope_table(oqn, positions, inv), max_ulp=2, frac_off=5e-2)
    check_close(to_np(k_rot), ORC.rope_table(okn, positions, inv), max_ulp=2, frac_off=5e-2)


def test_inv_freq_tables_match_oracle():
    from runtherder_b200.rope_tables import rope_inv_freq_llama3, rope_inv_freq_plain
    from runtherder_b200.configs import RopeScaling
    for D, theta in [(128, 500000.0), (64, 1.0e4), (256, 1.0e6), (128, 1.0e6)]:
        assert np.array_equal(rope_inv_freq_plain(D, theta).view(np.uint32), ORC.inv_freq_plain(D, theta).view(np.uint32))
        a = rope_inv_freq_llama3(D, theta, RopeScaling())
        assert np.array_equal(a.view(np.uint32), ORC.inv_freq_llama3(D, theta, 32.0, 1.0, 4.0, 8192).view(np.uint32))


def test_synth_generators_match_oracle():
    from runtherder_b200 import synth
    to_dev, to_np = _gpu()
    cs = synth.outlier_channel_scale(3072, 0, synth.T_X)
    assert (cs == 20.0).sum() == 16 and (cs == 1.0).sum() == 3072 - 16
    n, start = 5 * 3072, 7 * 3072
    a = synth.normal_bf16(n, 0, synth.T_X, start=start, chan_scale=to_dev(cs), ncols=3072)
    assert np.array_equal(to_np(a), ORC.synth_normal(n, 0, synth.T_X, start, 1.0, cs, 3072))
    a = synth.normal_bf16(4096, 1, synth.T_TABLE, std=0.02)
    assert np.array_equal(to_np(a), ORC.synth_normal(4096, 1, synth.T_TABLE, 0, 0.02))
    u = synth.uniform_bf16(4096, 0, synth.T_G_ATTN, 0.5, 1.5)
    assert np.array_equal(to_np(u), ORC.synth_uniform(4096, 0, synth.T_G_ATTN, 0.5, 1.5))
    i = synth.ids_i32(4096, 0, synth.T_IDS, 128256, start=11)
    assert np.array_equal(to_np(i), ORC.synth_ids(4096, 0, synth.T_IDS, 128256, 11))
    f = bf16_to_f32(ORC.synth_normal(200000, 3, 9))
    assert abs(f.mean()) < 0.01 and abs(f.std() - 1.0) < 0.01
