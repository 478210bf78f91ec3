"""Builds ``lit_gpt_b200/lib/libb200gpt.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m lit_gpt_b200.build [--force]

The library has no torch dependency: plain ``extern "C"`` over the CUDA runtime (statically linked), so it is the
drop-in boundary described in include/b200gpt.h.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libb200gpt.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "b200gpt.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libb200gpt.so")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers() -> list[str]:
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [HEADER]


def library_is_current() -> bool:
    """True when the full library exists and is newer than every source and header."""
    return not _stale(LIB, sources() + _headers())


def build_library(force: bool = False, verbose: bool = False, sources_subset: tuple[str, ...] | None = None, out: str | None = None) -> str:
    """Build the full library, or -- with ``sources_subset`` (file names under csrc/) and ``out`` -- a library of those sources
    only.  Objects are shared between the two, so neither build repeats the other's compilations."""
    srcs = sources() if sources_subset is None else [os.path.join(CSRC, f) for f in sources_subset]
    LIB = out or globals()["LIB"]
    headers = _headers()
    if not force and not _stale(LIB, srcs + headers):
        return LIB
    nvcc = _nvcc()
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd), file=sys.stderr)
            subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = f"{LIB}.{os.getpid()}.tmp"   # link beside the target, then rename: a concurrent reader never sees half a library
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp, *objs]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
