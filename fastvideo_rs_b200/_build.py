"""Builds libfvsdpa.so (the CUDA kernels and their C ABI) in-tree with nvcc for sm_100a.

    python -m fastvideo_rs_b200._build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The shared library lands next to this file so that it
travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfvsdpa.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG.parent / "include" / "fv_sdpa.h"]
    return any(p.stat().st_mtime > t for p in deps if p.is_file())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source under csrc/ into libfvsdpa.so; returns its path."""
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "-I", str(PKG.parent / "include"), "-o", str(LIB)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(s) for s in sources()]
    cmd += ["-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfvsdpa.so")
    return LIB


def build_native_checker() -> Path:
    """Compile tests/native/sdpa_check (the torch-free bring-up checker)."""
    src = PKG.parent / "tests" / "native" / "sdpa_check.cu"
    out = src.with_suffix(".bin")
    if out.exists() and out.stat().st_mtime > max(src.stat().st_mtime, LIB.stat().st_mtime):
        return out
    cmd = [nvcc_path(), *ARCH_FLAGS, "-O2", "-std=c++17", "-o", str(out), str(src), f"-L{PKG}", "-lfvsdpa", "-ldl",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../fastvideo_rs_b200"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building sdpa_check")
    return out


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
    print(build_native_checker())
