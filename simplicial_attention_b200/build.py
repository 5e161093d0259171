"""Build the CUDA library in-tree with nvcc for sm_100a.

    python -m simplicial_attention_b200.build [--force] [--verbose]

Produces ``simplicial_attention_b200/libsa2.so`` (C ABI in ``include/sa2.h``).
nvcc cross-compiles without a GPU, so this also serves as the build check.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libsa2.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _inputs() -> list[str]:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(ROOT, "include", "sa2.h"))
    files.append(os.path.abspath(__file__))
    return files


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > t for f in _inputs())


def build(force: bool = False, verbose: bool = False, out: str = LIB, defines: tuple[str, ...] = ()) -> str:
    """Compile libsa2.so if it is missing or older than its sources.  ``out`` and ``defines`` make a second
    build beside it (the diagnostic build with wait accounting, see waitprof.py); such a build is always redone."""
    if out == LIB and not force and not is_stale():
        return LIB
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        *ARCH_FLAGS,
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "--expt-relaxed-constexpr", *["-D" + d for d in defines],
        "-o", out, *sources(),
    ]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr, file=sys.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
