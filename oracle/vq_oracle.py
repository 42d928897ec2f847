"""numpy front-end of the C oracle in ``vq_oracle.c`` (test infrastructure only).

``build()`` compiles the C file into ``oracle/_build/libvqoracle.so`` with the host C
compiler (OpenMP when the compiler has it); the functions below wrap the C entry points
with numpy arrays.  Reference lines are cited in the C file at each function.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "vq_oracle.c"
_OUT = _HERE / "_build" / "libvqoracle.so"
_lib = None

BLOCK = 128


def build(force: bool = False) -> Path:
    """Compile the oracle if the shared object is missing or older than its source."""
    if not force and _OUT.exists() and (not _SRC.exists() or _OUT.stat().st_mtime >= _SRC.stat().st_mtime):
        return _OUT
    _OUT.parent.mkdir(exist_ok=True)
    base = ["-O2", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-shared", "-o", str(_OUT), str(_SRC), "-lm"]
    tried = []
    for cc in ("/usr/bin/gcc", "gcc", os.environ.get("CC", "cc"), "cc"):
        for omp in (["-fopenmp"], []):
            cmd = [cc] + omp + base
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return _OUT
            tried.append((" ".join(cmd), r.stderr.strip()[-300:]))
    raise RuntimeError("could not compile the oracle:\n" + "\n".join(f"{c}\n  {e}" for c, e in tried))


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_OUT))
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


_c_int, _c_long, _c_double = ctypes.c_int, ctypes.c_long, ctypes.c_double


def num_threads() -> int:
    lib = _load()
    lib.vqo_num_threads.restype = ctypes.c_int
    return int(lib.vqo_num_threads())


def round_bf16(x):
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    x = _f32(x)
    out = np.empty_like(x)
    _load().vqo_round_bf16(_p(x), _p(out), _c_long(x.size))
    return out


def assign_codes(k, cb, bias=None):
    """k [B,Hkv,L,D], cb [Hkv,M,K,D], bias None|[Hkv,M,K] -> codes [B,Hkv,L,M] int32."""
    k, cb = _f32(k), _f32(cb)
    B, Hkv, L, D = k.shape
    H2, M, K, D2 = cb.shape
    assert H2 == Hkv and D2 == D
    bias = _f32(bias) if bias is not None else None
    codes = np.empty((B, Hkv, L, M), dtype=np.int32)
    _load().vqo_assign_codes(_p(k), _p(cb), _p(bias), _c_int(B), _c_int(Hkv), _c_long(L), _c_int(D), _c_int(M),
                             _c_int(K), _p(codes))
    return codes


def assign_margin(k, cb, codes, bias=None):
    """fp64 margin of each given code over the best other codeword, and max |score|."""
    k, cb, codes = _f32(k), _f32(cb), _i32(codes)
    B, Hkv, L, D = k.shape
    _, M, K, _ = cb.shape
    bias = _f32(bias) if bias is not None else None
    margin = np.empty((B, Hkv, L, M), dtype=np.float64)
    maxabs = np.empty((B, Hkv, L, M), dtype=np.float64)
    _load().vqo_assign_margin(_p(k), _p(cb), _p(bias), _p(codes), _c_int(B), _c_int(Hkv), _c_long(L), _c_int(D),
                              _c_int(M), _c_int(K), _p(margin), _p(maxabs))
    return margin, maxabs


def build_aggregates(codes, v, K, NB=None):
    """codes [B,Hkv,L,M], v [B,Hkv,L,D] -> cnt [B,Hkv,NB,M,K] i32, vsum [B,Hkv,NB,M,K,D] f32."""
    codes, v = _i32(codes), _f32(v)
    B, Hkv, L, M = codes.shape
    D = v.shape[-1]
    if NB is None:
        NB = L // BLOCK
    assert NB * BLOCK <= L
    cnt = np.empty((B, Hkv, NB, M, K), dtype=np.int32)
    vsum = np.empty((B, Hkv, NB, M, K, D), dtype=np.float32)
    _load().vqo_build_aggregates(_p(codes), _p(v), _c_int(B), _c_int(Hkv), _c_long(L), _c_int(D), _c_int(M),
                                 _c_int(K), _c_int(NB), _p(cnt), _p(vsum))
    return cnt, vsum


def attn_naive(q1, q2, k1, k3, v, cb, codes, window, scale=None, rows=None):
    """Naive per-query VQ attention (restates ops/attn_vq.py:308-333); out [B,Hq,L,D] f32.

    Rows outside ``rows = (row0, row1)`` are left as NaN.
    """
    q1, q2, k1, k3, v, cb, codes = _f32(q1), _f32(q2), _f32(k1), _f32(k3), _f32(v), _f32(cb), _i32(codes)
    B, Hq, L, D = q1.shape
    Hkv = k1.shape[1]
    _, M, K, _ = cb.shape
    scale = float(scale) if scale is not None else 1.0 / np.sqrt(D)
    row0, row1 = rows if rows is not None else (0, L)
    out = np.full((B, Hq, L, D), np.nan, dtype=np.float32)
    _load().vqo_attn_naive(_p(q1), _p(q2), _p(k1), _p(k3), _p(v), _p(cb), _p(codes), _c_int(B), _c_int(Hq),
                           _c_int(Hkv), _c_long(L), _c_int(D), _c_int(M), _c_int(K), _c_long(window),
                           _c_double(scale), _c_long(row0), _c_long(row1), _p(out))
    return out


def attn_agg(q1, q2, k1, k3, v, cb, cnt, vsum, window, scale=None, rows=None, return_lse=False):
    """Attention from per-block aggregates (the fast path's arithmetic, double precision)."""
    q1, q2, k1, k3, v, cb = _f32(q1), _f32(q2), _f32(k1), _f32(k3), _f32(v), _f32(cb)
    cnt, vsum = _i32(cnt), _f32(vsum)
    B, Hq, L, D = q1.shape
    Hkv = k1.shape[1]
    _, M, K, _ = cb.shape
    NB = cnt.shape[2]
    scale = float(scale) if scale is not None else 1.0 / np.sqrt(D)
    row0, row1 = rows if rows is not None else (0, L)
    out = np.full((B, Hq, L, D), np.nan, dtype=np.float32)
    lse = np.full((B, Hq, L), np.nan, dtype=np.float32) if return_lse else None
    _load().vqo_attn_agg(_p(q1), _p(q2), _p(k1), _p(k3), _p(v), _p(cb), _p(cnt), _p(vsum), _c_int(NB), _c_int(B),
                         _c_int(Hq), _c_int(Hkv), _c_long(L), _c_int(D), _c_int(M), _c_int(K), _c_long(window),
                         _c_double(scale), _c_long(row0), _c_long(row1), _p(out), _p(lse))
    return (out, lse) if return_lse else out


def decode(q1, q2, k1w, k3w, vw, cb, cnt, vsum, n_valid, n_bd, scale=None, use_far=True):
    """Single-query decode from a cache; q [B,Hq,D], windows [B,Hkv,Nwin,D], out [B,Hq,D]."""
    q1, q2, k1w, k3w, vw, cb = _f32(q1), _f32(q2), _f32(k1w), _f32(k3w), _f32(vw), _f32(cb)
    cnt, vsum = _i32(cnt), _f32(vsum)
    B, Hq, D = q1.shape
    _, Hkv, Nwin, _ = k1w.shape
    _, M, K, _ = cb.shape
    scale = float(scale) if scale is not None else 1.0 / np.sqrt(D)
    out = np.empty((B, Hq, D), dtype=np.float32)
    _load().vqo_decode(_p(q1), _p(q2), _p(k1w), _p(k3w), _p(vw), _p(cb), _p(cnt), _p(vsum), _c_int(B), _c_int(Hq),
                       _c_int(Hkv), _c_long(Nwin), _c_long(n_valid), _c_long(n_bd), _c_int(D), _c_int(M), _c_int(K),
                       _c_double(scale), _c_int(1 if use_far else 0), _p(out))
    return out


# --------------------------------------------------------------------------------------
# Rotary helpers (HF Llama half-split convention, as used at ops/attn_vq.py:55-64,296-299).

def rope_tables(n_pos, D, base=10000.0):
    inv = 1.0 / (base ** (np.arange(0, D, 2, dtype=np.float64) / D))
    ang = np.arange(n_pos, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=-1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rotate_half(x):
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def apply_rope(x, cos, sin, positions):
    """x [..., L, D]; positions [L] (or scalar broadcast)."""
    c, s = cos[positions], sin[positions]
    return (x * c + rotate_half(x) * s).astype(np.float32)
