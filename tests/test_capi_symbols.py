"""The native library loads without a GPU and exports every entry point include/rh_kernels.h declares,
plus the C++ functions with the reference's exact (mangled) signatures that runtherder's callers link to.
No compute call is made here."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

# Itanium-mangled names of the reference's kernel API (namespace runtherder::kernels), i.e. what
# src/model/supported/llama/*.cu, include/runtherder/engine/kv_cache.h and src/kernels/matmul.cu
# reference at link time.  Identical to the symbols the reference's own kernel objects define.
REFERENCE_CXX_SYMBOLS = [
    "_ZN10runtherder7kernels20rmsnorm_bf16_forwardEP13__nv_bfloat16PKS1_S4_iifP11CUstream_st",
    "_ZN10runtherder7kernels24rmsnorm_add_bf16_forwardEP13__nv_bfloat16S2_PKS1_S4_S4_iifP11CUstream_st",
    "_ZN10runtherder7kernels23quantize_per_token_int8EPaPfPK13__nv_bfloat16iiP11CUstream_st",
    "_ZN10runtherder7kernels15dequantize_w8a8EP13__nv_bfloat16PKiPKfPKS1_iiP11CUstream_st",
    "_ZN10runtherder7kernels15quantize_kv_fp8EP13__nv_fp8_e4m3PfPK13__nv_bfloat16PKiiiiP11CUstream_st",
    "_ZN10runtherder7kernels19swiglu_bf16_forwardEP13__nv_bfloat16PKS1_S4_iP11CUstream_st",
    "_ZN10runtherder7kernels9rope_bf16EP13__nv_bfloat16S2_PKiPKfiiiiP11CUstream_st",
    "_ZN10runtherder7kernels29embedding_lookup_bf16_forwardEP13__nv_bfloat16PKS1_PKiiiP11CUstream_st",
    "_ZN10runtherder7kernels23flash_decode_split_bf16EP13__nv_bfloat16PKS1_PK13__nv_fp8_e4m3S7_PKfS9_PfiPKiiiifP11CUstream_st",
    "_ZN10runtherder7kernels18flash_prefill_bf16EP13__nv_bfloat16PKS1_PK13__nv_fp8_e4m3S7_PKfS9_iPKiiiifP11CUstream_st",
]
# bias.cu does not compile in the reference as shipped, so no reference object defines this one
BIAS_CXX_SYMBOL = "_ZN10runtherder7kernels25qkv_bias_add_bf16_forwardEP13__nv_bfloat16S2_S2_PKS1_S4_S4_iiiP11CUstream_st"


def declared_entry_points(header="rh_kernels.h"):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rh_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    from runtherder_b200 import _lib
    names = declared_entry_points()
    assert len(names) >= 20
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} is declared in rh_kernels.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"
    assert _lib.lib.rh_version() >= 100
    assert _lib.lib.rh_status_string(2) == b"unsupported dimension"


def test_linear_library_loads_and_exports_every_declared_symbol():
    """librh_linear.so (the W8A8 linear wrapper; links cuBLASLt) against include/rh_linear.h."""
    from runtherder_b200 import linear
    names = declared_entry_points("rh_linear.h")
    assert "rh_linear_w8a8_prequantized" in names and len(names) >= 5
    for name in names:
        assert hasattr(linear.lib, name), f"{name} is declared in rh_linear.h but not exported"
    assert set(names) == set(linear.SIGNATURES), "ctypes signature table and header disagree"


def test_library_exports_reference_cxx_signatures():
    from runtherder_b200 import _lib
    for sym in REFERENCE_CXX_SYMBOLS + [BIAS_CXX_SYMBOL]:
        getattr(_lib.lib, sym)  # raises AttributeError when missing


def test_reference_objects_define_the_same_symbols():
    """Where the reference's kernels were compiled here, their defined symbols are exactly this list."""
    ref = ROOT / "oracle" / "_ref" / "libref_cuda.so"
    if not ref.exists():
        pytest.skip("libref_cuda.so not built")
    lib = C.CDLL(str(ref))
    for sym in REFERENCE_CXX_SYMBOLS:
        getattr(lib, sym)


def test_no_fallback_when_library_missing(tmp_path, monkeypatch):
    """The loader raises instead of falling back when the shared object is absent."""
    from runtherder_b200 import _lib
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "librh_kernels.so")
    with pytest.raises(ImportError):
        _lib._load()
