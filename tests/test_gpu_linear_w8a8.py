"""The W8A8 linear wrapper (librh_linear.so) against the reference's own Matmul::linear_w8a8
(src/kernels/matmul.cu:126-158, compiled unmodified with its quantisation kernels into
oracle/_ref/libref_matmul.so): INT8 GEMMs accumulate exactly in int32 whatever algorithm cuBLASLt picks,
so y must be byte-identical — both for the reference's call shape (quantise inside) and when the codes
and per-token scales come from this library's fused kernels, which is what removes the repeated
quantisation from a decoder layer."""
import pytest
import torch

from refgen import make_bf16_random

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from gpu_util import bits_equal, mismatch_count, to_dev
    from oracle_lib import load_ref_matmul
    from runtherder_b200 import kernels, linear
    ref = load_ref_matmul()
    if ref is None:
        pytest.skip("oracle/_ref/libref_matmul.so is not present")
    class E: pass
    e = E()
    e.ref, e.K, e.mm, e.eq, e.count, e.to_dev = ref, kernels, linear.Matmul(), bits_equal, mismatch_count, to_dev
    return e


def _weights(env, n, k, seed):
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))
    w_scale = env.to_dev(make_bf16_random(n, 0.02, seed + 1)).abs() + 0.001
    return w, w_scale.to(torch.bfloat16)


def _reference(env, x, w, w_scale, m, n, k):
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    q = torch.empty(m, k, dtype=torch.int8, device="cuda"); s = torch.empty(m, dtype=torch.float32, device="cuda")
    acc = torch.empty(m, n, dtype=torch.int32, device="cuda")
    env.ref.refmatmul_linear_w8a8(y.data_ptr(), x.data_ptr(), w.data_ptr(), w_scale.data_ptr(), q.data_ptr(), s.data_ptr(),
                                  acc.data_ptr(), m, n, k, None)
    torch.cuda.synchronize()
    return y, q, s, acc


@pytest.mark.parametrize("m,n,k", [(35, 3072, 3072), (35, 1024, 3072), (511, 8192, 3072), (511, 3072, 8192), (1, 3072, 8192),
                                   (7, 264, 1000)])
def test_linear_w8a8_matches_reference_matmul(env, m, n, k):
    x = env.to_dev(make_bf16_random(m * k, 2.0, 0xAB + m)).view(m, k)
    w, w_scale = _weights(env, n, k, 5)
    y0, q0, s0, acc0 = _reference(env, x, w, w_scale, m, n, k)
    y1 = torch.empty_like(y0); q1 = torch.empty_like(q0); s1 = torch.empty_like(s0); acc1 = torch.empty_like(acc0)
    env.mm.linear_w8a8(y1, x, w, w_scale, q1, s1, acc1, m, n, k)
    torch.cuda.synchronize()
    assert env.eq(q0, q1) and env.eq(s0, s1)
    assert env.eq(acc0, acc1), f"{env.count(acc0, acc1)} accumulators differ"
    assert env.eq(y0, y1), f"{env.count(y0, y1)} of {y0.numel()} outputs differ"


@pytest.mark.parametrize("T,H,I", [(35, 3072, 8192), (511, 3072, 8192)])
def test_fused_kernels_feed_the_gemm_without_requantising(env, T, H, I):
    """The layer's two quantised inputs as the fused kernels write them — norm + INT8 for q/k/v/gate/up,
    SwiGLU + INT8 for the down projection — go straight into rh_linear_w8a8_prequantized; the result equals
    the reference's norm -> linear_w8a8 (x3, re-quantising each time) and swiglu -> linear_w8a8 sequence."""
    from gpu_util import ref_cuda_or_skip
    rk = ref_cuda_or_skip()
    x = env.to_dev(make_bf16_random(T * H, 1.0, 11)).view(T, H)
    res = env.to_dev(make_bf16_random(T * H, 1.0, 12)).view(T, H)
    g = env.to_dev(make_bf16_random(H, 0.5, 13)) + 1.0
    g = g.to(torch.bfloat16)
    gate = env.to_dev(make_bf16_random(T * I, 3.0, 14)).view(T, I)
    up = env.to_dev(make_bf16_random(T * I, 1.0, 15)).view(T, I)
    # reference: rmsnorm_add -> three linears on `normed`; swiglu -> one linear on `act`
    normed, h = torch.empty_like(x), torch.empty_like(x)
    rk.rmsnorm_add_bf16_forward(normed, h, x, res, g, T, H, 1e-5)
    act = torch.empty_like(gate)
    rk.swiglu_bf16_forward(act, gate, up, T * I)
    # this library: one fused launch per distinct input, then the GEMMs
    q_n = torch.empty(T, H, dtype=torch.int8, device="cuda"); s_n = torch.empty(T, dtype=torch.float32, device="cuda")
    h1 = torch.empty_like(x)
    env.K.rmsnorm_add_quant_int8(q_n, s_n, h1, None, x, res, g, T, H, 1e-5)
    q_a = torch.empty(T, I, dtype=torch.int8, device="cuda"); s_a = torch.empty(T, dtype=torch.float32, device="cuda")
    env.K.swiglu_quant_int8(q_a, s_a, None, gate, up, T, I)
    assert env.eq(h, h1)
    for n_out, seed in ((3072, 21), (1024, 22), (1024, 23)):          # q, k, v projections
        w, w_scale = _weights(env, n_out, H, seed)
        y0, _, _, _ = _reference(env, normed, w, w_scale, T, n_out, H)
        y1 = torch.empty_like(y0); acc = torch.empty(T, n_out, dtype=torch.int32, device="cuda")
        env.mm.linear_w8a8_prequantized(y1, q_n, s_n, w, w_scale, acc, T, n_out, H)
        torch.cuda.synchronize()
        assert env.eq(y0, y1), f"n={n_out}: {env.count(y0, y1)} outputs differ"
    w, w_scale = _weights(env, H, I, 31)                                # down projection
    y0, _, _, _ = _reference(env, act, w, w_scale, T, H, I)
    y1 = torch.empty_like(y0); acc = torch.empty(T, H, dtype=torch.int32, device="cuda")
    env.mm.linear_w8a8_prequantized(y1, q_a, s_a, w, w_scale, acc, T, H, I)
    torch.cuda.synchronize()
    assert env.eq(y0, y1), f"down projection: {env.count(y0, y1)} outputs differ"


def test_linear_w8a8_argument_checks(env):
    from runtherder_b200._lib import RhError
    y = torch.empty(4, 8, dtype=torch.bfloat16, device="cuda"); q = torch.empty(4, 6, dtype=torch.int8, device="cuda")
    s = torch.empty(4, dtype=torch.float32, device="cuda"); w = torch.empty(8, 6, dtype=torch.int8, device="cuda")
    ws = torch.empty(8, dtype=torch.bfloat16, device="cuda"); acc = torch.empty(4, 8, dtype=torch.int32, device="cuda")
    with pytest.raises(RhError):
        env.mm.linear_w8a8_prequantized(y, q, s, w, ws, acc, 4, 8, 6)      # k not a multiple of 4 (matmul.cu:136)
    with pytest.raises(RhError):
        env.mm.linear_w8a8_prequantized(y, q, s, w, ws, acc, 0, 8, 8)
