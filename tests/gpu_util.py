"""Helpers for the GPU parity tests: numpy(bf16 bits) <-> torch, and `RefCuda`, the reference's own
CUDA kernels (oracle/_ref/libref_cuda.so) behind the reference's function names."""
from __future__ import annotations

import numpy as np
import torch

from oracle_lib import load_ref_cuda


def to_dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    """numpy -> cuda tensor; uint16 arrays are bf16 bit patterns."""
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda().view(torch.bfloat16)
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def to_np(t: torch.Tensor) -> np.ndarray:
    """cuda tensor -> numpy; bf16 comes back as uint16 bit patterns, fp8 as uint8."""
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).cpu().numpy()
    return t.cpu().numpy()


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bitwise equality on the device (NaNs with equal payload compare equal)."""
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    w = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[a.element_size()]
    return bool(torch.equal(a.contiguous().view(w), b.contiguous().view(w)))


def mismatch_count(a: torch.Tensor, b: torch.Tensor) -> int:
    w = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[a.element_size()]
    return int((a.contiguous().view(w) != b.contiguous().view(w)).sum().item())


def _s(stream):
    if stream is None:
        return torch.cuda.current_stream().cuda_stream or None
    return int(stream) or None


class RefCudaUnavailable(RuntimeError):
    pass


def ref_cuda_or_skip():
    """RefCuda() for a test: skips (instead of failing) where the checker cannot exist."""
    import pytest
    try:
        return RefCuda()
    except RefCudaUnavailable as exc:
        pytest.skip(str(exc))


class _RefCallPlan:
    def __init__(self, owner):
        self.owner, self.calls = owner, []

    def __getattr__(self, name):        # stands in for the ctypes library while recording
        fn = getattr(self.owner._real_lib, name)

        def recorded(*args):
            self.calls.append((fn, args))
            return fn(*args)
        return recorded

    def __enter__(self):
        self.owner.lib = self
        return self

    def __exit__(self, *exc):
        self.owner.lib = self.owner._real_lib

    def replay(self):
        for fn, args in self.calls:
            fn(*args)
        return len(self.calls)


class RefCuda:
    """The reference's kernels, callable with torch tensors under the reference's names."""

    def __init__(self):
        self.lib = load_ref_cuda()
        if self.lib is None:   # a checkout without the reference's sources and without the prebuilt checker
            raise RefCudaUnavailable("oracle/_ref/libref_cuda.so is not present and the reference's sources "
                                     "are not available to build it")
        self._real_lib = self.lib

    def record(self):
        """Context manager: the calls made inside are executed and also recorded; the returned object's
        replay() issues them again with the same pointers and sizes, skipping the tensor-to-pointer
        conversions (the launch cost a C++ caller of the reference's kernels sees)."""
        return _RefCallPlan(self)

    def rmsnorm_bf16_forward(self, y, x, g, T, H, eps, stream=None):
        self.lib.refcuda_rmsnorm(y.data_ptr(), x.data_ptr(), g.data_ptr(), T, H, eps, _s(stream))

    def rmsnorm_add_bf16_forward(self, y, h_out, x, residual, g, T, H, eps, stream=None):
        self.lib.refcuda_rmsnorm_add(y.data_ptr(), h_out.data_ptr(), x.data_ptr(), residual.data_ptr(),
                                     g.data_ptr(), T, H, eps, _s(stream))

    def quantize_per_token_int8(self, q, x_scale, x, T, K, stream=None):
        self.lib.refcuda_quantize_per_token_int8(q.data_ptr(), x_scale.data_ptr(), x.data_ptr(), T, K, _s(stream))

    def dequantize_w8a8(self, y, acc, x_scale, w_scale, m, n, stream=None):
        self.lib.refcuda_dequantize_w8a8(y.data_ptr(), acc.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(), m, n,
                                         _s(stream))

    def quantize_kv_fp8(self, q, scale, x, at_pos, rows_per_pos, num_rows, D, stream=None):
        self.lib.refcuda_quantize_kv_fp8(q.data_ptr(), scale.data_ptr(), x.data_ptr(), at_pos.data_ptr(),
                                         rows_per_pos, num_rows, D, _s(stream))

    def swiglu_bf16_forward(self, y, gate, up, n, stream=None):
        self.lib.refcuda_swiglu(y.data_ptr(), gate.data_ptr(), up.data_ptr(), n, _s(stream))

    def rope_bf16(self, q, k, positions, inv_freq, T, Hq, Hkv, D, stream=None):
        self.lib.refcuda_rope(q.data_ptr(), k.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(), T, Hq, Hkv, D,
                              _s(stream))

    def embedding_lookup_bf16_forward(self, out, table, ids, T, H, stream=None):
        self.lib.refcuda_embedding_lookup(out.data_ptr(), table.data_ptr(), ids.data_ptr(), T, H, _s(stream))

    def attention_causal_bf16(self, out, q, k, v, k_scale, v_scale, n_new, cache_len, Hq, Hkv, D, scale, stream=None):
        self.lib.refcuda_attention_causal(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), k_scale.data_ptr(),
                                          v_scale.data_ptr(), n_new, cache_len.data_ptr(), Hq, Hkv, D, scale, _s(stream))

    def flash_prefill_bf16(self, out, q, k, v, k_scale, v_scale, n_new, cache_len, Hq, Hkv, D, scale, stream=None):
        self.lib.refcuda_flash_prefill(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), k_scale.data_ptr(),
                                       v_scale.data_ptr(), n_new, cache_len.data_ptr(), Hq, Hkv, D, scale, _s(stream))

    def flash_decode_split_bf16(self, out, q, k, v, k_scale, v_scale, partial, num_splits, cache_len, Hq, Hkv, D, scale,
                                stream=None):
        self.lib.refcuda_flash_decode_split(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                            k_scale.data_ptr(), v_scale.data_ptr(), partial.data_ptr(), num_splits,
                                            cache_len.data_ptr(), Hq, Hkv, D, scale, _s(stream))
