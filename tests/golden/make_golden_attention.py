"""Generates tests/golden/reference_cuda_attention.npz from the REFERENCE ITSELF: its naive causal attention
(src/kernels/attention.cu — the oracle of its own flash tests) and its flash_decode_split_bf16
(src/kernels/flash_decode.cu) and flash_prefill_bf16 (src/kernels/flash_prefill.cu), compiled unmodified for
sm_100a into oracle/_ref/libref_cuda.so by oracle/Makefile, run on a B200 at the decode shape (n_new = 1) and
at small prefill shapes over a few seeded caches.  The
reference has no host implementation of attention, so these GPU outputs are what pins the CPU oracle
(orc_attention_decode_fp8) when no GPU is present.

Needs a CUDA device, the built library and oracle/_ref:
    python tests/golden/make_golden_attention.py [output.npz]
Inputs (q bits, cache codes, scales) and both kernels' outputs are stored whole; a case is a few KB.
"""
import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))
from gpu_util import RefCuda, to_np  # noqa: E402

# (cache_len, q heads, kv heads, head_dim, splits, q multiplier)
CASES = [(40, 8, 2, 64, 4, 1.0), (0, 4, 2, 32, 1, 1.0), (97, 6, 2, 128, 8, 6.0), (33, 4, 4, 64, 3, 3.0), (130, 14, 2, 32, 5, 2.0)]
# (n_new, cache_len, q heads, kv heads, q multiplier), head_dim 128
PREFILL_CASES = [(20, 0, 8, 2, 1.0), (8, 10, 6, 2, 4.0), (33, 5, 4, 4, 2.0)]


def main() -> None:
    from runtherder_b200 import kernels as K
    ref = RefCuda()
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE / "reference_cuda_attention.npz"
    arrays = {"cases": np.array(CASES, np.float64)}
    for idx, (cache_len, Hq, Hkv, D, splits, q_mul) in enumerate(CASES):
        g = torch.Generator(device="cuda").manual_seed(1000 + idx)
        n = cache_len + 1
        q = ((torch.rand(Hq, D, device="cuda", generator=g) * 2 - 1) * q_mul).to(torch.bfloat16)
        k = (torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
        v = (torch.randn(n, Hkv, D, device="cuda", generator=g) * torch.exp(torch.randn(n, Hkv, 1, device="cuda", generator=g))).to(torch.bfloat16)
        at = torch.zeros(1, dtype=torch.int32, device="cuda")
        kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda"); vc = torch.empty_like(kc)
        ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda"); vs = torch.empty_like(ks)
        ref.quantize_kv_fp8(kc, ks, k, at, 1, n * Hkv, D)          # the reference's own cache writer
        ref.quantize_kv_fp8(vc, vs, v, at, 1, n * Hkv, D)
        cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
        scale = 1.0 / math.sqrt(D)
        naive = torch.empty(Hq, D, dtype=torch.bfloat16, device="cuda")
        split = torch.empty_like(naive)
        part = torch.empty(K.flash_split_scratch_floats(Hq, D, splits), dtype=torch.float32, device="cuda")
        ref.attention_causal_bf16(naive, q, kc, vc, ks, vs, 1, cl, Hq, Hkv, D, scale)
        ref.flash_decode_split_bf16(split, q, kc, vc, ks, vs, part, splits, cl, Hq, Hkv, D, scale)
        torch.cuda.synchronize()
        for name, t in (("q", q), ("k_codes", kc), ("v_codes", vc), ("k_scale", ks), ("v_scale", vs),
                        ("out_naive", naive), ("out_split", split)):
            arrays[f"case{idx}/{name}"] = to_np(t)
    # prefill shapes (n_new > 1): the reference's naive kernel and its flash_prefill_bf16 (head_dim 128 only)
    arrays["prefill_cases"] = np.array(PREFILL_CASES, np.float64)
    for idx, (n_new, cache_len, Hq, Hkv, q_mul) in enumerate(PREFILL_CASES):
        D = 128
        g = torch.Generator(device="cuda").manual_seed(2000 + idx)
        n = cache_len + n_new
        q = ((torch.rand(n_new, Hq, D, device="cuda", generator=g) * 2 - 1) * q_mul).to(torch.bfloat16)
        k = (torch.rand(n, Hkv, D, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
        v = (torch.randn(n, Hkv, D, device="cuda", generator=g) * torch.exp(torch.randn(n, Hkv, 1, device="cuda", generator=g))).to(torch.bfloat16)
        at = torch.zeros(1, dtype=torch.int32, device="cuda")
        kc = torch.empty(n, Hkv, D, dtype=torch.uint8, device="cuda"); vc = torch.empty_like(kc)
        ks = torch.empty(n, Hkv, dtype=torch.float32, device="cuda"); vs = torch.empty_like(ks)
        ref.quantize_kv_fp8(kc, ks, k, at, 1, n * Hkv, D)
        ref.quantize_kv_fp8(vc, vs, v, at, 1, n * Hkv, D)
        cl = torch.tensor([cache_len], dtype=torch.int32, device="cuda")
        naive = torch.empty(n_new, Hq, D, dtype=torch.bfloat16, device="cuda")
        flash = torch.empty_like(naive)
        ref.attention_causal_bf16(naive, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 1.0 / math.sqrt(D))
        ref.flash_prefill_bf16(flash, q, kc, vc, ks, vs, n_new, cl, Hq, Hkv, D, 1.0 / math.sqrt(D))
        torch.cuda.synchronize()
        for name, t in (("q", q), ("k_codes", kc), ("v_codes", vc), ("k_scale", ks), ("v_scale", vs),
                        ("out_naive", naive), ("out_flash", flash)):
            arrays[f"prefill{idx}/{name}"] = to_np(t)
    np.savez_compressed(out_path, **arrays)
    print(f"wrote {out_path} ({out_path.stat().st_size} bytes, {len(CASES)} decode + {len(PREFILL_CASES)} prefill cases)")


if __name__ == "__main__":
    main()
