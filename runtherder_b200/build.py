"""Builds librh_kernels.so in-tree with nvcc for sm_100a.

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

SOURCES = ["capi.cu", "rows.cu", "swiglu.cu", "rope_kv.cu", "embedding.cu", "flash_decode.cu", "flash_prefill.cu", "flash_prefill_tc.cu", "synth.cu", "dropin.cu", "selftest_static.cu"]

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
    if force or _stale(LIB, objs):
        cmd = [cc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of librh_kernels.so failed")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
