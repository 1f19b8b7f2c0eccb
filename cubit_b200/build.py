"""Builds libcubit_b200.so (CUDA kernels + C ABI) in-tree for sm_100a.

Usage: ``python -m cubit_b200.build [--force] [--verbose]``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import fcntl
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB = LIB_DIR / "libcubit_b200.so"
SOURCES = ["capi.cu", "isa_table.cpp", "flat_table.cpp", "elf_text.cpp", "sass_text.cpp", "sass_print.cpp"]
HEADERS = ["codec_core.cuh", "flat_table.hpp", "isa_table.hpp", "elf_text.hpp", "sass_text.hpp", "json.hpp",
           "../../include/cubit_b200.h"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library if it is missing or older than its sources; returns its path.

    Several processes may call this at once (one rank per GPU under torchrun): one of them compiles, into a file of
    its own that takes the library's name only when it is complete, and the others wait for it."""
    if not force and not is_stale():
        return LIB
    LIB_DIR.mkdir(exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():      # another process built it while this one waited
                return LIB
            tmp = LIB_DIR / f".libcubit_b200.{os.getpid()}.so"
            cmd = [nvcc_path(), "-O3", "-std=c++17", "-lineinfo", *ARCH, "-shared", "-Xcompiler",
                   "-fPIC,-Wall,-Wno-unused-function,-Wno-unknown-pragmas", "-cudart", "static", "-o", str(tmp)] \
                  + [str(CSRC / s) for s in SOURCES] + ["-ldl", "-lpthread"]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), file=sys.stderr)
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
            if verbose:
                print(proc.stdout + proc.stderr, file=sys.stderr)
            os.replace(tmp, LIB)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
