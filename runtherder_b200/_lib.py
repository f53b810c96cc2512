"""ctypes binding of librh_kernels.so (the C ABI declared in include/rh_kernels.h).

The library is the only implementation: if it is missing or fails to load, importing
this module raises.  There is no PyTorch or CPU fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "_C" / "librh_kernels.so"

RH_OK = 0
STATUS_NAMES = {0: "RH_OK", 1: "RH_ERR_INVALID_ARG", 2: "RH_ERR_UNSUPPORTED_DIM", 3: "RH_ERR_MISALIGNED",
                4: "RH_ERR_LAUNCH", 5: "RH_ERR_CUDA"}

_p, _i, _f = C.c_void_p, C.c_int, C.c_float
_ll, _sz, _u64, _i32 = C.c_longlong, C.c_size_t, C.c_uint64, C.c_int32

# name -> argtypes; every function returns int unless listed in _RESTYPES
SIGNATURES = {
    "rh_version": [],
    "rh_init": [_i],
    "rh_status_string": [_i],
    "rh_last_error_string": [],
    "rh_rmsnorm_bf16": [_p, _p, _p, _i, _i, _f, _p],
    "rh_rmsnorm_add_bf16": [_p, _p, _p, _p, _p, _i, _i, _f, _p],
    "rh_rmsnorm_add_last_row_bf16": [_p, _p, _p, _p, _i, _i, _f, _p],
    "rh_quantize_per_token_int8": [_p, _p, _p, _i, _i, _p],
    "rh_dequantize_w8a8": [_p, _p, _p, _p, _i, _i, _p],
    "rh_quantize_kv_fp8": [_p, _p, _p, _p, _i, _i, _i, _p],
    "rh_swiglu_bf16": [_p, _p, _p, _ll, _p],
    "rh_rope_bf16": [_p, _p, _p, _p, _i, _i, _i, _i, _p],
    "rh_embedding_lookup_bf16": [_p, _p, _p, _i, _i, _p],
    "rh_qkv_bias_add_bf16": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p],
    "rh_flash_split_scratch_floats": [_i, _i, _i],
    "rh_flash_decode_split_bf16": [_p, _p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _p],
    "rh_flash_prefill_bf16": [_p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _p],
    "rh_rmsnorm_add_quant_int8": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p],
    "rh_swiglu_quant_int8": [_p, _p, _p, _p, _p, _i, _i, _p],
    "rh_rope_kv_fp8": [_p, _p, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "rh_bias_rope_kv_fp8": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "rh_stage_positions": [_p, _p, _i, _i, _p],
    "rh_decode_advance": [_p, _p, _p, _p, _i, _p],
    "rh_rope_inv_freq_plain": [_p, _i, _f],
    "rh_rope_inv_freq_llama3": [_p, _i, _f, _f, _f, _f, _i],
    "rh_synth_normal_bf16": [_p, _sz, _u64, _u64, _u64, _f, _p, _i, _p],
    "rh_synth_uniform_bf16": [_p, _sz, _u64, _u64, _u64, _f, _f, _p],
    "rh_synth_ids_i32": [_p, _sz, _u64, _u64, _u64, _i32, _p],
    "rh_tune": [C.c_char_p, _i],
    "rh_selftest": [_p],
    "rh_device_error": [_p],
    "rh_selfcheck_bounded_wait": [_i, _p, _p],
    "rh_selfcheck_role_wait": [_i, _p],
    "rh_selftest_static": [_p, _i, _p],
}
_RESTYPES = {"rh_status_string": C.c_char_p, "rh_last_error_string": C.c_char_p,
             "rh_flash_split_scratch_floats": C.c_size_t}


class RhError(RuntimeError):
    """A C-ABI call returned a non-zero rh_status."""

    def __init__(self, fn: str, status: int, message: str):
        self.fn, self.status, self.message = fn, status, message
        super().__init__(f"{fn}: {STATUS_NAMES.get(status, status)}: {message}")


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m runtherder_b200.build` "
            "(needs nvcc; the package has no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is stale
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int)
    return lib


lib = _load()


_recording = None   # the call list of the active CallPlan, if any


class CallPlan:
    """Records the C-ABI calls made inside its `with` block (they are executed as usual) and replays them:
    the same entry points with the same pointers, sizes and stream, without the Python mirror's argument
    checks in between — the launch cost a C++ caller of the library sees.  Only valid while the tensors whose
    addresses were recorded are alive and for the stream that was current when it was recorded."""

    def __init__(self):
        self.calls = []

    def __enter__(self):
        global _recording
        if _recording is not None:
            raise RuntimeError("a CallPlan is already recording")
        _recording = self.calls
        return self

    def __exit__(self, *exc):
        global _recording
        _recording = None

    def replay(self) -> int:
        """Issues every recorded call again; returns how many were issued."""
        for fn, name, args in self.calls:
            status = fn(*args)
            if status != RH_OK:
                raise RhError(name, status, lib.rh_last_error_string().decode())
        return len(self.calls)


def call(name: str, *args) -> None:
    """Invoke an rh_* entry point and raise RhError on a non-zero status."""
    fn = getattr(lib, name)
    if _recording is not None:
        _recording.append((fn, name, args))
    status = fn(*args)
    if status != RH_OK:
        raise RhError(name, status, lib.rh_last_error_string().decode())
