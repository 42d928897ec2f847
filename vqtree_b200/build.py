"""Builds the CUDA library (``vqtree_b200/lib/libvqattn.so``) for sm_100a with nvcc, in-tree.

    python -m vqtree_b200.build [--force] [--verbose]

The shared object exports only the C ABI declared in ``include/vqattn.h``.  It is not a Python
extension: the host layer binds it with ctypes, any other host language can bind it the same way.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "build"
LIB = LIBDIR / "libvqattn.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
SOURCES = ["api.cu", "assign.cu", "assign_tc.cu", "aggregate.cu", "aggregate_reg.cu", "prefill_simt.cu", "prefill_tc4.cu", "rope.cu", "decode.cu", "decode_bulk.cu", "decode_tc.cu"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = nvcc_path()
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    flags = ARCH + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", str(ROOT / "include"), "-I", str(CSRC)]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: str):
        s = CSRC / src
        o = OBJDIR / (s.stem + ".o")
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + flags + ["-c", str(s), "-o", str(o)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
        return o

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _stale(LIB, objs):
        cmd = [nvcc] + ARCH + ["-shared", "-o", str(LIB)] + [str(o) for o in objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
