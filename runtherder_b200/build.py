"""Builds librh_kernels.so (the kernels) and librh_linear.so (the W8A8 linear wrapper, which adds the
cuBLASLt dependency) in-tree with nvcc for sm_100a.

Usage: python -m runtherder_b200.build [--force] [--verbose]

The library is placed in runtherder_b200/_C/ so that it travels with the source
tree; nothing is installed into site-packages and nothing is JIT-compiled at
import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_C"
INCLUDE = PKG.parent / "include"
LIB = OUT / "librh_kernels.so"
LINEAR_LIB = OUT / "librh_linear.so"
LINEAR_SOURCES = ["linear_w8a8.cu"]

SOURCES = ["capi.cu", "rows.cu", "swiglu.cu", "rope_kv.cu", "embedding.cu", "flash_decode.cu", "flash_prefill.cu", "flash_prefill_tc.cu", "flash_prefill_ws.cu", "synth.cu", "dropin.cu", "selftest_static.cu"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=default",
    "-Xptxas", "-warn-spills",
]


def nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; librh_kernels.so cannot be built")
    return cand


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + list(INCLUDE.glob("*.hpp"))
    cc = nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> Path:
        obj = OUT / (src.rsplit(".", 1)[0] + ".o")
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [cc, *NVCC_FLAGS, *extra, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(CSRC / src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
        linear_objs = list(pool.map(compile_one, LINEAR_SOURCES))
    if force or _stale(LIB, objs):
        cmd = [cc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of librh_kernels.so failed")
    if force or _stale(LINEAR_LIB, linear_objs + [LIB]):
        # The wrapper resolves the kernels from librh_kernels.so beside it and cuBLASLt from the process
        # (a Python process that imported torch has libcublasLt.so.12 mapped already) or the CUDA toolkit.
        cuda_lib = str(Path(cc).resolve().parent.parent / "lib64")
        cmd = [cc, "-shared", "-o", str(LINEAR_LIB), *map(str, linear_objs), f"-L{OUT}", "-lrh_kernels",
               f"-L{cuda_lib}", "-lcublasLt", "-cudart", "static",
               "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", f"-rpath={cuda_lib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of librh_linear.so failed")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
