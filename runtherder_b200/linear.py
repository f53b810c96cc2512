"""The W8A8 linear layer around the fused quantisation kernels (librh_linear.so; C ABI in
include/rh_linear.h).  Mirrors runtherder::kernels::Matmul for the INT8 path
(include/runtherder/kernels/matmul.cuh:36-71): `Matmul.linear_w8a8` is the reference's call (quantise x,
INT8 GEMM, dequantise), `Matmul.linear_w8a8_prequantized` takes codes and per-token scales that a fused
kernel already produced.  The GEMM is cuBLASLt, as in the reference.  No fallback: importing this
module raises when the shared library is missing."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

from ._lib import RhError, lib as _kernels   # librh_kernels.so must be mapped first (librh_linear.so links it)
from .kernels import _stream

LIB_PATH = Path(__file__).resolve().parent / "_C" / "librh_linear.so"

_p, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
SIGNATURES = {
    "rh_linear_w8a8_prequantized": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p, _p, _sz, _p],
    "rh_linear_w8a8": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p, _p, _sz, _p],
    "rh_linear_create_handle": [C.POINTER(_p)],
    "rh_linear_destroy_handle": [_p],
    "rh_linear_release": [_p],
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m runtherder_b200.build`")
    lib = C.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    return lib


lib = _load()


def _call(name: str, *args) -> None:
    status = getattr(lib, name)(*args)
    if status != 0:
        raise RhError(name, status, _kernels.rh_last_error_string().decode())


class Matmul:
    """A cuBLASLt handle and a 32 MiB workspace (the reference's kWorkspaceBytes, matmul.cuh:133), built once."""

    WORKSPACE_BYTES = 32 << 20

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        with torch.cuda.device(self.device):
            handle = _p()
            _call("rh_linear_create_handle", C.byref(handle))
            self.handle = handle
            self.workspace = torch.empty(self.WORKSPACE_BYTES, dtype=torch.uint8, device=self.device)

    def close(self) -> None:
        if self.handle is not None:
            _call("rh_linear_destroy_handle", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def linear_w8a8_prequantized(self, y, q, x_scale, weight, w_scale, acc, m, n, k, stream=None) -> None:
        """y[m,n] = bf16((q . weight^T) * x_scale[row] * w_scale[col]); q [m,k] int8, weight [n,k] int8,
        acc [m,n] int32 scratch."""
        _call("rh_linear_w8a8_prequantized", y.data_ptr(), q.data_ptr(), x_scale.data_ptr(), weight.data_ptr(),
              w_scale.data_ptr(), acc.data_ptr(), m, n, k, self.handle, self.workspace.data_ptr(),
              self.WORKSPACE_BYTES, _stream(stream))

    def linear_w8a8(self, y, x, weight, w_scale, q, x_scale, acc, m, n, k, stream=None) -> None:
        """The reference's Matmul::linear_w8a8: x [m,k] bf16 is quantised into q / x_scale first."""
        _call("rh_linear_w8a8", y.data_ptr(), x.data_ptr(), weight.data_ptr(), w_scale.data_ptr(), q.data_ptr(),
              x_scale.data_ptr(), acc.data_ptr(), m, n, k, self.handle, self.workspace.data_ptr(),
              self.WORKSPACE_BYTES, _stream(stream))
