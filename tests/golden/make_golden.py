"""Generates tests/golden/reference_host.npz and reference_host_digests.json from the REFERENCE
ITSELF: the host-side helpers of its kernel tests (rmsnorm_cpu_reference,
rmsnorm_add_cpu_reference, quantize_kv_reference, rope_cpu_reference, swiglu_cpu_reference,
make_bf16_random) and CUDA's host number-format conversions, compiled unmodified into
oracle/_ref/libref_host.so by oracle/Makefile.  Cases and seeds are the reference tests' own
(tests/kernels/test_{rmsnorm,quantization,rope,activation}.cpp).

Run where the reference sources are available:  python tests/golden/make_golden.py
Small cases are stored whole (inputs and outputs); every case also gets SHA-256 digests.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
from oracle_lib import load_ref_host, ptr  # noqa: E402

STORE_LIMIT = 24 * 1024  # elements; larger cases are kept as digests only


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ref = load_ref_host()
    if ref is None:
        raise SystemExit("reference sources not available: cannot regenerate golden vectors")
    arrays, digests = {}, {}

    def rnd(count, scale, seed):
        out = np.empty(count, np.uint16)
        ref.refhost_make_bf16_random(ptr(out), count, scale, seed)
        return out

    def put(case, **kw):
        digests[case] = {k: sha(v) for k, v in kw.items()}
        if max(v.size for v in kw.values()) <= STORE_LIMIT:
            for k, v in kw.items():
                arrays[f"{case}/{k}"] = v

    # number formats: CUDA's host conversions
    rng = np.random.default_rng(20240607)
    bits = np.concatenate([
        rng.integers(0, 2 ** 32, 6000, dtype=np.uint64).astype(np.uint32),
        (np.arange(0, 65536, 37, dtype=np.uint32) << 16) | 0x8000,   # exact ties
        (np.arange(0, 65536, 41, dtype=np.uint32) << 16) | 0x7fff,
        np.array([0x7f800000, 0xff800000, 0x7fc00000, 0x7f800001, 0, 0x80000000, 1, 0x007fffff], np.uint32)])
    f = bits.view(np.float32)
    arrays["formats/f32_bits"] = bits
    arrays["formats/bf16"] = np.array([ref.refhost_f32_to_bf16(float(v)) for v in f], np.uint16)
    e_in = np.concatenate([
        rng.uniform(-500, 500, 3000), rng.uniform(-2, 2, 2000), rng.uniform(-0.02, 0.02, 2000),
        [448, 449, 463.99, 464, 464.01, 480, 1e9, -1e9, np.inf, -np.inf, np.nan, 2.0 ** -9, 2.0 ** -10,
         1.5 * 2.0 ** -10, 2.0 ** -10 * 1.0000001, 0.0, -0.0, 2.0 ** -6, 2.0 ** -6 - 2.0 ** -11],
        np.arange(0, 32, 0.0625), -np.arange(0, 480, 3.5)]).astype(np.float32)
    arrays["formats/e4m3_in"] = e_in
    arrays["formats/e4m3"] = np.array([ref.refhost_f32_to_e4m3(float(v)) for v in e_in], np.uint8)
    arrays["formats/e4m3_decode"] = np.array([ref.refhost_e4m3_to_f32(b) for b in range(256)], np.float32)

    eps = 1e-5
    for T, H in [(1, 128), (4, 2560), (2, 16384), (32, 2560)]:          # test_rmsnorm.cpp:211-241
        x, g = rnd(T * H, 1.0, 0xC0FFEE), rnd(H, 0.5, 0xBADBEEF)
        y = np.empty_like(x)
        ref.refhost_rmsnorm(ptr(y), ptr(x), ptr(g), T, H, eps)
        put(f"rmsnorm_{T}x{H}", x=x, g=g, y=y)
        x, r, g = rnd(T * H, 1.0, 0xFEEDFACE), rnd(T * H, 1.0, 0xDEADBEEF), rnd(H, 0.5, 0xCAFEBABE)
        y, h = np.empty_like(x), np.empty_like(x)
        ref.refhost_rmsnorm_add(ptr(y), ptr(h), ptr(x), ptr(r), ptr(g), T, H, eps)
        put(f"rmsnorm_add_{T}x{H}", x=x, residual=r, g=g, y=y, h_out=h)

    for R, D, seed in [(24, 128, 0xC0FFEE), (8, 256, 0xBADBEEF), (512, 128, 0xFEEDFACE)]:  # test_quantization.cpp:126-136
        x = rnd(R * D, 1.0, seed)
        q, s = np.empty(R * D, np.uint8), np.empty(R, np.float32)
        ref.refhost_quantize_kv(ptr(q), ptr(s), ptr(x), R, D)
        put(f"kvfp8_{R}x{D}", x=x, q=q, scale=s)
    x = np.zeros(2 * 128, np.uint16)                                       # test_quantization.cpp:138-170
    q, s = np.empty(2 * 128, np.uint8), np.empty(2, np.float32)
    ref.refhost_quantize_kv(ptr(q), ptr(s), ptr(x), 2, 128)
    put("kvfp8_zero_2x128", x=x, q=q, scale=s)

    for T, Hq, Hkv, D, theta, pos in [(1, 4, 1, 64, 1.0e4, 0), (8, 32, 8, 128, 1.0e6, 0), (1, 32, 8, 128, 1.0e6, 1024),
                                      (2, 8, 2, 256, 1.0e6, 0), (32, 32, 8, 128, 1.0e6, 0)]:  # test_rope.cpp:186-205
        q, k = rnd(T * Hq * D, 1.0, 0xC0FFEE), rnd(T * Hkv * D, 1.0, 0xBADBEEF)
        qo, ko = q.copy(), k.copy()
        ref.refhost_rope(ptr(qo), pos, T, Hq, D, theta)
        ref.refhost_rope(ptr(ko), pos, T, Hkv, D, theta)
        put(f"rope_T{T}_q{Hq}_kv{Hkv}_D{D}_pos{pos}", q=q, k=k, q_out=qo, k_out=ko)

    for n, sg, su in [(128, 0xC0FFEE, 0xBADBEEF), (9728, 0xC0FFEE, 0xBADBEEF), (8 * 9728, 0xC0FFEE, 0xBADBEEF),
                      (32 * 9728, 0xC0FFEE, 0xBADBEEF), (4 * 9728, 0x12345, 0x67890)]:   # test_activation.cpp:106-150
        g, u = rnd(n, 2.0, sg), rnd(n, 2.0, su)
        y = np.empty_like(g)
        ref.refhost_swiglu(ptr(y), ptr(g), ptr(u), n)
        put(f"swiglu_n{n}_seed{sg:x}", gate=g, up=u, y=y)

    for n, q_dim, kv_dim in [(3, 64, 16), (1, 1536, 256), (511, 2048, 256)]:             # test_bias.cpp:103-116
        for name, dim, sx, sb in (("q", q_dim, 0x1111, 0x4444), ("k", kv_dim, 0x2222, 0x5555), ("v", kv_dim, 0x3333, 0x6666)):
            x, b = rnd(n * dim, 4.0, sx), rnd(dim, 2.0, sb)
            out = np.empty_like(x)
            ref.refhost_add_rows(ptr(out), ptr(x), ptr(b), n, dim)
            put(f"bias_{name}_n{n}_dim{dim}", x=x, bias=b, out=out)

    np.savez_compressed(HERE / "reference_host.npz", **arrays)
    (HERE / "reference_host_digests.json").write_text(json.dumps(digests, indent=1, sort_keys=True) + "\n")
    print(f"{len(arrays)} arrays, {len(digests)} cases")


if __name__ == "__main__":
    main()
