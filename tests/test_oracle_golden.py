"""The C oracle against golden vectors produced by the reference's own host helpers and CUDA's host
number-format conversions (tests/golden/make_golden.py).  Bit-exact everywhere: the oracle restates
the same double/float arithmetic."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from oracle_lib import Oracle, load_ref_host, ptr
from refgen import f32_to_bf16, make_bf16_random

GOLD = Path(__file__).resolve().parent / "golden"
ARR = np.load(GOLD / "reference_host.npz")
DIG = json.loads((GOLD / "reference_host_digests.json").read_text())
ORC = Oracle()


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_bf16_conversion_matches_cuda_host():
    f = ARR["formats/f32_bits"].view(np.float32)
    got = np.array([ORC.lib.orc_f32_to_bf16(float(v)) for v in f], np.uint16)
    assert np.array_equal(got, ARR["formats/bf16"])
    assert np.array_equal(f32_to_bf16(f), ARR["formats/bf16"])  # the numpy helper used by the tests too


def test_e4m3_conversion_matches_cuda_host():
    got = np.array([ORC.lib.orc_f32_to_e4m3(float(v)) for v in ARR["formats/e4m3_in"]], np.uint8)
    assert np.array_equal(got, ARR["formats/e4m3"])
    dec = np.array([ORC.lib.orc_e4m3_to_f32(b) for b in range(256)], np.float32)
    np.testing.assert_array_equal(dec, ARR["formats/e4m3_decode"])  # NaN == NaN here


def _inputs(case, names, gen):
    """Stored inputs when the case is small, else regenerated with the reference tests' generator and
    checked against the stored digest."""
    out = []
    for name, (count, scale, seed) in zip(names, gen):
        key = f"{case}/{name}"
        a = ARR[key] if key in ARR.files else make_bf16_random(count, scale, seed)
        assert sha(a) == DIG[case][name], f"{case}: input {name} differs from the reference generator"
        out.append(a)
    return out


@pytest.mark.parametrize("T,H", [(1, 128), (4, 2560), (2, 16384), (32, 2560)])
def test_rmsnorm_matches_reference_host(T, H):
    case = f"rmsnorm_{T}x{H}"
    x, g = _inputs(case, ["x", "g"], [(T * H, 1.0, 0xC0FFEE), (H, 0.5, 0xBADBEEF)])
    y = ORC.rmsnorm(x.reshape(T, H), g, 1e-5)
    assert sha(y) == DIG[case]["y"]


@pytest.mark.parametrize("T,H", [(1, 128), (4, 2560), (2, 16384), (32, 2560)])
def test_rmsnorm_add_matches_reference_host(T, H):
    case = f"rmsnorm_add_{T}x{H}"
    x, r, g = _inputs(case, ["x", "residual", "g"],
                      [(T * H, 1.0, 0xFEEDFACE), (T * H, 1.0, 0xDEADBEEF), (H, 0.5, 0xCAFEBABE)])
    y, h = ORC.rmsnorm_add(x.reshape(T, H), r.reshape(T, H), g, 1e-5)
    assert sha(h) == DIG[case]["h_out"]
    assert sha(y) == DIG[case]["y"]


@pytest.mark.parametrize("R,D,seed", [(24, 128, 0xC0FFEE), (8, 256, 0xBADBEEF), (512, 128, 0xFEEDFACE)])
def test_kv_fp8_matches_reference_host(R, D, seed):
    case = f"kvfp8_{R}x{D}"
    (x,) = _inputs(case, ["x"], [(R * D, 1.0, seed)])
    q, s = ORC.quant_kv(x.reshape(R, D))
    assert sha(q) == DIG[case]["q"]
    assert sha(s) == DIG[case]["scale"]


def test_kv_fp8_zero_rows():
    q, s = ORC.quant_kv(np.zeros((2, 128), np.uint16))
    assert sha(q) == DIG["kvfp8_zero_2x128"]["q"] and not q.any()
    assert sha(s) == DIG["kvfp8_zero_2x128"]["scale"] and not s.any()


def test_kv_fp8_slot_addressing():
    """dst_row = row + at_pos*rows_per_pos (src/kernels/quantization.cu:210-211): the rows land in the
    slab where a [slots, rows_per_pos, D] cache keeps position at_pos, and nothing else is touched."""
    x = make_bf16_random(3 * 8 * 128, 1.0, 7).reshape(24, 128)
    q0, s0 = ORC.quant_kv(x)
    q, s = ORC.quant_kv(x, at_pos=5, rows_per_pos=8, slots=10 * 8)
    assert np.array_equal(q[40:64], q0) and np.array_equal(s[40:64], s0)
    assert not q[:40].any() and not q[64:].any() and not s[:40].any() and not s[64:].any()


@pytest.mark.parametrize("T,Hq,Hkv,D,theta,pos", [(1, 4, 1, 64, 1.0e4, 0), (8, 32, 8, 128, 1.0e6, 0),
                                                   (1, 32, 8, 128, 1.0e6, 1024), (2, 8, 2, 256, 1.0e6, 0),
                                                   (32, 32, 8, 128, 1.0e6, 0)])
def test_rope_matches_reference_host(T, Hq, Hkv, D, theta, pos):
    case = f"rope_T{T}_q{Hq}_kv{Hkv}_D{D}_pos{pos}"
    q, k = _inputs(case, ["q", "k"], [(T * Hq * D, 1.0, 0xC0FFEE), (T * Hkv * D, 1.0, 0xBADBEEF)])
    assert sha(ORC.rope_theta(q.reshape(T, Hq, D), pos, theta)) == DIG[case]["q_out"]
    assert sha(ORC.rope_theta(k.reshape(T, Hkv, D), pos, theta)) == DIG[case]["k_out"]
    # the table-driven variant (how the kernel is fed) stays within the reference tests' tolerance of it
    from oracle_lib import bf16_to_f32
    pos_arr = np.arange(pos, pos + T, dtype=np.int32)
    tab = ORC.rope_table(q.reshape(T, Hq, D), pos_arr, ORC.inv_freq_plain(D, theta))
    assert np.abs(bf16_to_f32(tab) - bf16_to_f32(ORC.rope_theta(q.reshape(T, Hq, D), pos, theta))).max() <= 5e-2


@pytest.mark.parametrize("n,sg,su", [(128, 0xC0FFEE, 0xBADBEEF), (9728, 0xC0FFEE, 0xBADBEEF),
                                     (8 * 9728, 0xC0FFEE, 0xBADBEEF), (32 * 9728, 0xC0FFEE, 0xBADBEEF),
                                     (4 * 9728, 0x12345, 0x67890)])
def test_swiglu_matches_reference_host(n, sg, su):
    case = f"swiglu_n{n}_seed{sg:x}"
    g, u = _inputs(case, ["gate", "up"], [(n, 2.0, sg), (n, 2.0, su)])
    assert sha(ORC.swiglu(g, u)) == DIG[case]["y"]


@pytest.mark.parametrize("n,q_dim,kv_dim", [(3, 64, 16), (1, 1536, 256), (511, 2048, 256)])
def test_bias_add_matches_reference_host(n, q_dim, kv_dim):
    for name, dim, sx, sb in (("q", q_dim, 0x1111, 0x4444), ("k", kv_dim, 0x2222, 0x5555), ("v", kv_dim, 0x3333, 0x6666)):
        case = f"bias_{name}_n{n}_dim{dim}"
        x, b = _inputs(case, ["x", "bias"], [(n * dim, 4.0, sx), (dim, 2.0, sb)])
        assert sha(ORC.add_rows(x.reshape(n, dim), b)) == DIG[case]["out"]


def test_inv_freq_known_answers():
    """Values of theta^(-2i/D) and of the Llama-3 rescaling computed independently from the formula
    (src/model/supported/llama/llama.cu:128-143, llama3.cu:26-60) for the benchmark configurations."""
    f = ORC.inv_freq_llama3(128, 500000.0, 32.0, 1.0, 4.0, 8192).view(np.uint32)
    assert [hex(f[i]) for i in (1, 28, 29, 32, 34, 35, 63)] == [
        "0x3f508ac1", "0x3b527720", "0x3b0ad4f9", "0x39e13623", "0x38cb98f8", "0x37c86886", "0x33a4c2ff"]
    plain = ORC.inv_freq_plain(128, 500000.0)
    assert np.array_equal(f[:29], plain.view(np.uint32)[:29])          # short wavelengths untouched
    assert np.allclose(f[35:].view(np.float32) * 32.0, plain[35:], rtol=1e-6)  # long ones divided by factor
    q = ORC.inv_freq_plain(128, 1.0e6)
    assert q[0] == 1.0 and float(q[1]) == 0.8058421611785889 and float(q[32]) == 0.0010000000474974513
    assert float(q[63]) == 1.2409377632138785e-06


def test_int8_quant_properties():
    """quantize_per_token_int8 has no host code in the reference; pin the restatement of
    src/kernels/quantization.cu:63-96 through its defining properties."""
    x = make_bf16_random(64 * 3072, 3.0, 11).reshape(64, 3072)
    x[5] = 0                                        # zero row -> scale 0, codes 0
    q, s = ORC.quant_int8(x)
    from oracle_lib import bf16_to_f32
    xf = bf16_to_f32(x)
    amax = np.abs(xf).max(axis=1)
    assert np.array_equal(s, (amax / np.float32(127.0)).astype(np.float32))
    assert s[5] == 0 and not q[5].any()
    assert np.abs(q.astype(np.int32)).max() == 127 and q.min() >= -127
    live = amax > 0
    inv = np.zeros_like(amax)
    inv[live] = np.float32(127.0) / amax[live]
    expect = np.clip(np.rint((xf * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(q, expect)
    # ties go to even: x*inv == 0.5 exactly -> 0, 1.5 -> 2
    row = np.zeros(8, np.float32); row[0] = 127.0; row[1] = 0.5; row[2] = 1.5; row[3] = -2.5
    qt, st = ORC.quant_int8(f32_to_bf16(row).reshape(1, 8))
    assert st[0] == 1.0 and list(qt[0][:4]) == [127, 0, 2, -2]


def test_embedding_and_dequant_restatements():
    rng = np.random.default_rng(3)
    table = rng.integers(0, 65536, (100, 64), dtype=np.uint16)
    ids = rng.integers(0, 100, 17, dtype=np.int32)
    assert np.array_equal(ORC.embedding(table, ids), table[ids])
    acc = rng.integers(-50000, 50000, (5, 12), dtype=np.int32)
    xs = rng.uniform(0.001, 0.1, 5).astype(np.float32)
    ws = f32_to_bf16(rng.uniform(0.001, 0.05, 12).astype(np.float32))
    from oracle_lib import bf16_to_f32
    expect = f32_to_bf16(((acc.astype(np.float32) * xs[:, None]).astype(np.float32) * bf16_to_f32(ws)[None, :]))
    assert np.array_equal(ORC.dequant_w8a8(acc, xs, ws), expect)


def test_reference_input_generator_port():
    """refgen.make_bf16_random == the reference tests' make_bf16_random (checked live when the compiled
    reference helpers are present, and through the stored digests above in any case)."""
    ref = load_ref_host()
    if ref is None:
        pytest.skip("compiled reference helpers not present")
    for count, scale, seed in [(1000, 1.0, 0xC0FFEE), (777, 0.5, 0xBADBEEF), (4096, 2.0, 0x12345)]:
        out = np.empty(count, np.uint16)
        ref.refhost_make_bf16_random(ptr(out), count, scale, seed)
        assert np.array_equal(out, make_bf16_random(count, scale, seed))


def test_oracle_matches_compiled_reference_live():
    """When libref_host.so is present, compare on fresh random shapes as well (not only the stored cases)."""
    ref = load_ref_host()
    if ref is None:
        pytest.skip("compiled reference helpers not present")
    x, r, g = (make_bf16_random(7 * 1032, 1.5, s) for s in (1, 2, 3))
    g = g[:1032]
    y, h = np.empty_like(x), np.empty_like(x)
    ref.refhost_rmsnorm_add(ptr(y), ptr(h), ptr(x), ptr(r), ptr(g), 7, 1032, 1e-6)
    oy, oh = ORC.rmsnorm_add(x.reshape(7, 1032), r.reshape(7, 1032), g, 1e-6)
    assert np.array_equal(oy.ravel(), y) and np.array_equal(oh.ravel(), h)
    gate, up = make_bf16_random(5000, 6.0, 4), make_bf16_random(5000, 6.0, 5)
    out = np.empty_like(gate)
    ref.refhost_swiglu(ptr(out), ptr(gate), ptr(up), 5000)
    assert np.array_equal(ORC.swiglu(gate, up), out)
    t = make_bf16_random(3 * 5 * 96, 1.0, 6)
    tt = t.copy()
    ref.refhost_rope(ptr(tt), 40000, 3, 5, 96, 500000.0)
    assert np.array_equal(ORC.rope_theta(t.reshape(3, 5, 96), 40000, 500000.0).ravel(), tt)


def test_attention_oracle_is_within_one_ulp_of_the_reference_kernels():
    """The reference has no host attention; its naive kernel (the oracle of its flash tests) and its split
    decode kernel were run on a B200 by tests/golden/make_golden_attention.py.  The double-precision
    restatement must round to within one bf16 ulp of both on every element that is not a cancellation
    residue, and within 1.5 * 2^-7 of the row maximum everywhere."""
    data = np.load(GOLD / "reference_cuda_attention.npz")
    cases = data["cases"]
    assert len(cases) >= 5

    def ordered(bits):
        b = bits.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)

    for idx, (cache_len, Hq, Hkv, D, _splits, _q_mul) in enumerate(cases):
        cache_len, D = int(cache_len), int(D)
        g = lambda name: np.ascontiguousarray(data[f"case{idx}/{name}"])
        bits, exact = ORC.attention_decode_fp8(g("q"), g("k_codes"), g("v_codes"), g("k_scale"), g("v_scale"),
                                               cache_len, 1.0 / np.sqrt(np.float32(D)).item())
        rowmax = np.abs(exact).max(axis=1, keepdims=True)
        significant = np.abs(exact) >= rowmax / 64
        for name in ("out_naive", "out_split"):
            ref_bits = g(name)
            ref_val = (ref_bits.astype(np.uint32) << 16).view(np.float32)
            assert (np.abs(ref_val - exact) <= 1.5 * 2.0 ** -7 * rowmax).all(), (idx, name)
            assert np.abs(ordered(ref_bits) - ordered(bits))[significant].max() <= 1, (idx, name)
            assert (ordered(ref_bits) == ordered(bits)).mean() > 0.99, (idx, name)


def test_prefill_oracle_is_within_one_ulp_of_the_reference_naive_kernel():
    """n_new > 1: the reference's naive causal kernel (run on a B200 by make_golden_attention.py) is the oracle of
    its flash_prefill test; the double-precision restatement must round to within one bf16 ulp of it.  The
    reference's flash_prefill kernel, which rounds its operands to f16, must stay within its own test's bounds
    of the restatement (max-abs 5e-2 at this value range, cosine 0.998: tests/kernels/test_flash_prefill.cpp:88-89)."""
    data = np.load(GOLD / "reference_cuda_attention.npz")
    cases = data["prefill_cases"]
    assert len(cases) >= 3

    def ordered(bits):
        b = bits.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)

    for idx, (n_new, cache_len, Hq, Hkv, _q_mul) in enumerate(cases):
        g = lambda name: np.ascontiguousarray(data[f"prefill{idx}/{name}"])
        bits, exact = ORC.attention_causal_fp8(g("q"), g("k_codes"), g("v_codes"), g("k_scale"), g("v_scale"),
                                               int(cache_len), 1.0 / np.sqrt(np.float32(128)).item())
        rowmax = np.abs(exact).max(axis=-1, keepdims=True)
        significant = np.abs(exact) >= rowmax / 64
        naive = g("out_naive")
        assert np.abs(ordered(naive) - ordered(bits))[significant].max() <= 1, idx
        assert (ordered(naive) == ordered(bits)).mean() > 0.99, idx
        flash = (g("out_flash").astype(np.uint32) << 16).view(np.float32).ravel().astype(np.float64)
        e = exact.ravel().astype(np.float64)
        assert np.dot(flash, e) / (np.linalg.norm(flash) * np.linalg.norm(e)) >= 0.998, idx
        assert (np.abs(flash - e) <= 1.5 * 2.0 ** -7 * np.repeat(rowmax.ravel(), 128) * 4).all(), idx
