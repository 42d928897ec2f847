"""Builds the CUDA library (``vqtree_b200/lib/libvqattn.so``) for sm_100a with nvcc, in-tree.

    python -m vqtree_b200.build [--force] [--verbose]

The shared object exports only the C ABI declared in ``include/vqattn.h``.  It is not a Python
extension: the host layer binds it with ctypes, any other host language can bind it the same way.
``build_torch_ext`` compiles the PyTorch C++ extension over that ABI (``lib/libvqattn_torch.so``:
``csrc/torch_ext.cpp``, host code only, g++ against the installed torch headers), which registers the
entry points as ``torch.ops.vqattn.*``.
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


TORCH_EXT = LIBDIR / "libvqattn_torch.so"


def build_torch_ext(force: bool = False, verbose: bool = False) -> Path:
    """g++ build of csrc/torch_ext.cpp against the installed torch; links libvqattn.so from the same folder."""
    import torch
    from torch.utils import cpp_extension
    lib = build(force=False, verbose=verbose)
    src = CSRC / "torch_ext.cpp"
    if not force and not _stale(TORCH_EXT, [src, lib, ROOT / "include" / "vqattn.h"]):
        return TORCH_EXT
    # The system compiler, whose libstdc++ is the shared one the process already runs on.  ($CXX may name a
    # toolchain that links its own libstdc++ statically into the extension: that private copy's stream locale is
    # never initialised, and formatting an error message through it crashes.)
    cxx = next((c for c in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")) if c and Path(c).exists()), "g++")
    cuda_home = os.environ.get("CUDA_HOME") or str(Path(nvcc_path()).resolve().parent.parent)
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-unknown-pragmas",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + [str(Path(cuda_home) / "include"), str(ROOT / "include")]:
        cmd += ["-isystem" if "torch" in inc or "cuda" in inc else "-I", inc]
    cmd += [str(src), "-o", str(TORCH_EXT), f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            f"-L{LIBDIR}", "-lvqattn", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("g++ failed on torch_ext.cpp")
    nm = shutil.which("nm")
    if nm:   # a statically linked libstdc++ shows as thousands of std:: definitions in the dynamic symbol table
        syms = subprocess.run([nm, "-D", "--defined-only", str(TORCH_EXT)], capture_output=True, text=True).stdout
        if "_ZNSo9_M_insertIlEERSoT_" in syms:
            TORCH_EXT.unlink()
            raise RuntimeError(f"{cxx} linked libstdc++ statically into the extension; build it with the system g++")
    return TORCH_EXT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    print(build_torch_ext(a.force, a.verbose))
