"""ctypes bindings of the checkers: oracle/_build/liboracle.so (the C restatement),
oracle/_ref/libref_host.so (the reference's own host helpers) and oracle/_ref/libref_cuda.so
(the reference's own CUDA kernels built for sm_100a).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

import os

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
# Where the reference's sources lie when they are present at all (the checkers under oracle/_ref are
# built from them in place): a checkout named `reference` beside this repository, or wherever REF points,
# exactly as for oracle/Makefile.
REFERENCE_ROOT = Path(os.environ.get("REF", str(ROOT.parent / "reference")))

_p, _i, _f, _l = C.c_void_p, C.c_int, C.c_float, C.c_long
_sz, _u64, _u32, _i32, _u16, _u8 = C.c_size_t, C.c_uint64, C.c_uint32, C.c_int32, C.c_uint16, C.c_uint8


def _make(target: str) -> None:
    subprocess.run(["make", "-C", str(ORACLE_DIR), f"REF={REFERENCE_ROOT}", target], check=True, capture_output=True)


def load_oracle() -> C.CDLL:
    path = ORACLE_DIR / "_build" / "liboracle.so"
    src = ORACLE_DIR / "rh_oracle.c"
    if not path.exists() or path.stat().st_mtime < src.stat().st_mtime:
        _make("oracle")
    lib = C.CDLL(str(path))
    sig = {
        "orc_bf16_to_f32": ([_u16], _f), "orc_f32_to_bf16": ([_f], _u16),
        "orc_f32_to_e4m3": ([_f], _u8), "orc_e4m3_to_f32": ([_u8], _f),
        "orc_dequantize_kv_fp8": ([_u8, _f], _f),
        "orc_rmsnorm": ([_p, _p, _p, _l, _i, _f], None),
        "orc_rmsnorm_add": ([_p, _p, _p, _p, _p, _l, _i, _f, _p], None),
        "orc_quantize_per_token_int8": ([_p, _p, _p, _l, _i], None),
        "orc_dequantize_w8a8": ([_p, _p, _p, _p, _l, _i], None),
        "orc_quantize_kv_fp8": ([_p, _p, _p, _i, _i, _l, _i], None),
        "orc_swiglu": ([_p, _p, _p, _sz], None),
        "orc_add_rows": ([_p, _p, _p, _l, _i], None),
        "orc_rope_theta": ([_p, _i, _l, _i, _i, _f], None),
        "orc_rope_table": ([_p, _p, _p, _l, _i, _i], None),
        "orc_rope_inv_freq_plain": ([_p, _i, _f], None),
        "orc_rope_inv_freq_llama3": ([_p, _i, _f, _f, _f, _f, _i], None),
        "orc_embedding_lookup": ([_p, _p, _p, _l, _i], None),
        "orc_rmsnorm_add_quant_int8": ([_p, _p, _p, _p, _p, _p, _p, _l, _i, _f, _p], None),
        "orc_swiglu_quant_int8": ([_p, _p, _p, _p, _p, _l, _i], None),
        "orc_rope_kv_fp8": ([_p, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _i, _l, _i, _i, _i], None),
        "orc_attention_decode_fp8": ([_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _p], None),
        "orc_attention_causal_fp8": ([_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p], None),
        "orc_synth_normal_bf16": ([_p, _sz, _u64, _u64, _u64, _f, _p, _i], None),
        "orc_synth_uniform_bf16": ([_p, _sz, _u64, _u64, _u64, _f, _f], None),
        "orc_synth_ids_i32": ([_p, _sz, _u64, _u64, _u64, _i32], None),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    return lib


def ref_host_path() -> Path:
    return ORACLE_DIR / "_ref" / "libref_host.so"


def ref_cuda_path() -> Path:
    return ORACLE_DIR / "_ref" / "libref_cuda.so"


def load_ref_host():
    """The reference's host helpers; None when neither the prebuilt library nor the reference sources exist."""
    path = ref_host_path()
    if not path.exists():
        if not REFERENCE_ROOT.exists():
            return None
        _make("_ref/libref_host.so")
    lib = C.CDLL(str(path))
    sig = {
        "refhost_rmsnorm": ([_p, _p, _p, _i, _i, _f], C.c_double),
        "refhost_rmsnorm_add": ([_p, _p, _p, _p, _p, _i, _i, _f], C.c_double),
        "refhost_make_bf16_random": ([_p, _sz, _f, _u32], None),
        "refhost_f32_to_bf16": ([_f], _u16), "refhost_bf16_to_f32": ([_u16], _f),
        "refhost_f32_to_e4m3": ([_f], _u8), "refhost_e4m3_to_f32": ([_u8], _f),
        "refhost_quantize_kv": ([_p, _p, _p, _i, _i], C.c_double),
        "refhost_dequantize_kv_fp8": ([_u8, _f], _f),
        "refhost_rope": ([_p, _i, _i, _i, _i, _f], C.c_double),
        "refhost_swiglu": ([_p, _p, _p, _sz], C.c_double),
        "refhost_add_rows": ([_p, _p, _p, _i, _i], None),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    return lib


def load_ref_cuda():
    """The reference's CUDA kernels (sm_100a); None when the prebuilt library is absent."""
    path = ref_cuda_path()
    if not path.exists():
        if not REFERENCE_ROOT.exists():
            return None
        _make("_ref/libref_cuda.so")
    lib = C.CDLL(str(path))
    sig = {
        "refcuda_rmsnorm": [_p, _p, _p, _i, _i, _f, _p],
        "refcuda_rmsnorm_add": [_p, _p, _p, _p, _p, _i, _i, _f, _p],
        "refcuda_quantize_per_token_int8": [_p, _p, _p, _i, _i, _p],
        "refcuda_dequantize_w8a8": [_p, _p, _p, _p, _i, _i, _p],
        "refcuda_quantize_kv_fp8": [_p, _p, _p, _p, _i, _i, _i, _p],
        "refcuda_swiglu": [_p, _p, _p, _i, _p],
        "refcuda_rope": [_p, _p, _p, _p, _i, _i, _i, _i, _p],
        "refcuda_embedding_lookup": [_p, _p, _p, _i, _i, _p],
        "refcuda_attention_causal": [_p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _p],
        "refcuda_flash_decode_split": [_p, _p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _p],
        "refcuda_flash_prefill": [_p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _p],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, None
    return lib


def load_ref_matmul():
    """The reference's W8A8 linear layer (matmul.cu + cuBLASLt); None when the prebuilt library is absent."""
    path = ORACLE_DIR / "_ref" / "libref_matmul.so"
    if not path.exists():
        if not REFERENCE_ROOT.exists():
            return None
        _make("_ref/libref_matmul.so")
    lib = C.CDLL(str(path))
    lib.refmatmul_linear_w8a8.argtypes = [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]
    lib.refmatmul_linear_w8a8.restype = None
    return lib


def ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    """numpy front end of liboracle.so; bf16 tensors are uint16 arrays, FP8 uint8."""

    def __init__(self):
        self.lib = load_oracle()

    def rmsnorm(self, x, g, eps):
        T, H = x.shape
        y = np.empty_like(x)
        self.lib.orc_rmsnorm(ptr(y), ptr(x), ptr(g), T, H, eps)
        return y

    def rmsnorm_add(self, x, res, g, eps):
        T, H = x.shape
        y, h = np.empty_like(x), np.empty_like(x)
        tmp = np.empty(H, np.float32)
        self.lib.orc_rmsnorm_add(ptr(y), ptr(h), ptr(x), ptr(res), ptr(g), T, H, eps, ptr(tmp))
        return y, h

    def quant_int8(self, x):
        T, K = x.shape
        q, s = np.empty((T, K), np.int8), np.empty(T, np.float32)
        self.lib.orc_quantize_per_token_int8(ptr(q), ptr(s), ptr(x), T, K)
        return q, s

    def dequant_w8a8(self, acc, x_scale, w_scale):
        m, n = acc.shape
        y = np.empty((m, n), np.uint16)
        self.lib.orc_dequantize_w8a8(ptr(y), ptr(acc), ptr(x_scale), ptr(w_scale), m, n)
        return y

    def quant_kv(self, x, at_pos=0, rows_per_pos=1, slots=None):
        R, D = x.shape
        total = at_pos * rows_per_pos + R if slots is None else slots
        q, s = np.zeros((total, D), np.uint8), np.zeros(total, np.float32)
        self.lib.orc_quantize_kv_fp8(ptr(q), ptr(s), ptr(x), at_pos, rows_per_pos, R, D)
        return q, s

    def attention_decode_fp8(self, q, k, v, k_scale, v_scale, cache_len, scale):
        """q [Hq, D] bf16 bits; k, v [n, Hkv, D] uint8 codes; scales [n, Hkv] -> (bf16 bits, float32) [Hq, D]."""
        Hq, D = q.shape
        Hkv = k.shape[1]
        out = np.empty((Hq, D), np.uint16)
        out_f = np.empty((Hq, D), np.float32)
        buf = np.empty(cache_len + 1, np.float64)
        self.lib.orc_attention_decode_fp8(ptr(out), ptr(out_f), ptr(q), ptr(k), ptr(v), ptr(k_scale), ptr(v_scale),
                                          cache_len, Hq, Hkv, D, scale, ptr(buf))
        return out, out_f

    def attention_causal_fp8(self, q, k, v, k_scale, v_scale, cache_len, scale):
        """q [n_new, Hq, D] bf16 bits; k, v [cache_len + n_new, Hkv, D] codes -> (bf16 bits, float32) [n_new, Hq, D]."""
        n_new, Hq, D = q.shape
        Hkv = k.shape[1]
        out = np.empty((n_new, Hq, D), np.uint16)
        out_f = np.empty((n_new, Hq, D), np.float32)
        buf = np.empty(cache_len + n_new, np.float64)
        self.lib.orc_attention_causal_fp8(ptr(out), ptr(out_f), ptr(q), ptr(k), ptr(v), ptr(k_scale), ptr(v_scale),
                                          n_new, cache_len, Hq, Hkv, D, scale, ptr(buf))
        return out, out_f

    def add_rows(self, x, bias):
        n, dim = x.shape
        out = np.empty_like(x)
        self.lib.orc_add_rows(ptr(out), ptr(x), ptr(bias), n, dim)
        return out

    def swiglu(self, gate, up):
        y = np.empty_like(gate)
        self.lib.orc_swiglu(ptr(y), ptr(gate), ptr(up), gate.size)
        return y

    def rope_theta(self, t, start_pos, theta):
        T, Hh, D = t.shape
        out = t.copy()
        self.lib.orc_rope_theta(ptr(out), start_pos, T, Hh, D, theta)
        return out

    def rope_table(self, t, positions, inv_freq):
        T, Hh, D = t.shape
        out = t.copy()
        self.lib.orc_rope_table(ptr(out), ptr(positions), ptr(inv_freq), T, Hh, D)
        return out

    def inv_freq_plain(self, D, theta):
        out = np.empty(D // 2, np.float32)
        self.lib.orc_rope_inv_freq_plain(ptr(out), D, theta)
        return out

    def inv_freq_llama3(self, D, theta, factor, low, high, orig):
        out = np.empty(D // 2, np.float32)
        self.lib.orc_rope_inv_freq_llama3(ptr(out), D, theta, factor, low, high, orig)
        return out

    def embedding(self, table, ids):
        out = np.empty((ids.size, table.shape[1]), np.uint16)
        self.lib.orc_embedding_lookup(ptr(out), ptr(table), ptr(ids), ids.size, table.shape[1])
        return out

    def synth_normal(self, count, seed, tid, start=0, std=1.0, chan_scale=None, ncols=1):
        out = np.empty(count, np.uint16)
        self.lib.orc_synth_normal_bf16(ptr(out), count, seed, tid, start, std,
                                       None if chan_scale is None else ptr(chan_scale), ncols)
        return out

    def synth_uniform(self, count, seed, tid, lo, hi, start=0):
        out = np.empty(count, np.uint16)
        self.lib.orc_synth_uniform_bf16(ptr(out), count, seed, tid, start, lo, hi)
        return out

    def synth_ids(self, count, seed, tid, modulus, start=0):
        out = np.empty(count, np.int32)
        self.lib.orc_synth_ids_i32(ptr(out), count, seed, tid, start, modulus)
        return out


def bf16_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << 16).view(np.float32)


def bf16_ulp_diff(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in bf16 units in the last place between two uint16 bf16 arrays."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7fff), u & 0x7fff)
    return np.abs(key(a) - key(b))
