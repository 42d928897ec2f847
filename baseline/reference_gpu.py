"""The reference's own GPU path, timed on this machine (the side arm ``bench.py --impl reference-gpu``).

Loads the reference's files from ``baseline/_ref/ops`` (placed there by ``baseline/install_ref.py``; never
committed) without importing its package ``__init__`` (which needs a transformers API the installed release
no longer has): ``mini_vq.py`` and the two Triton kernel files are loaded by path; the host preparation
``long_prefilling_sort_based_linear`` is a method of a ``LlamaAttention`` subclass that cannot be imported, so
its source is parsed out of ``attn_vq.py`` and executed against a small stand-in ``self`` (rotary tables in the
HF Llama half-split convention).  The kernels, the wrapper ``vq_attn_forward`` (local kernel, far kernel,
flashinfer merge) and the host preparation are the reference's, unmodified.

Limits of the reference that shape the workload: ONE codebook per head ([H, C, D]), no grouped-query heads,
sequence length a multiple of 128 (its log-sum-exp store is not masked on a ragged last tile,
ops/triton_fused_local_attn_rerope.py:214-216), counts cast to the 16-bit activation dtype
(ops/attn_vq.py:432), so C is chosen such that counts stay exactly representable.
"""
from __future__ import annotations

import ast
import importlib.util
import math
import os
import sys
import textwrap
import types
from functools import partial
from pathlib import Path

import torch

REF = Path(__file__).resolve().parent / "_ref"

# The reference's kernels read a plain module-level constant (NEGINF) from inside @triton.jit code, which Triton 3
# refuses unless this switch is on; it is Triton's own documented way to run such kernels unmodified.
os.environ.setdefault("TRITON_ALLOW_NON_CONSTEXPR_GLOBALS", "1")


def available():
    need = ("mini_vq.py", "attn_vq.py", "triton_fused_vq_attn.py", "triton_fused_local_attn_rerope.py")
    missing = [f for f in need if not (REF / "ops" / f).exists()]
    return (not missing), ("baseline/_ref/ops lacks " + ", ".join(missing) + " (run baseline/install_ref.py)" if missing else "")


def load_modules():
    try:
        import triton
        triton.knobs.compilation.allow_non_constexpr_globals = True
    except Exception:
        pass
    pkg = types.ModuleType("ops")
    pkg.__path__ = [str(REF / "ops")]
    sys.modules["ops"] = pkg
    mods = {}
    for name in ("mini_vq", "triton_fused_local_attn_rerope", "triton_fused_vq_attn"):
        spec = importlib.util.spec_from_file_location(f"ops.{name}", REF / "ops" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"ops.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def extract_method(name: str) -> str:
    src = (REF / "ops" / "attn_vq.py").read_text()
    for node in ast.parse(src).body:
        if isinstance(node, ast.ClassDef) and node.name == "LlamaFlashAttention2VectorQuantizedReRoPE":
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and item.name == name:
                    return textwrap.dedent(ast.get_source_segment(src, item))
    raise KeyError(name)


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids, unsqueeze_dim=1):
    cos, sin = cos[position_ids].unsqueeze(unsqueeze_dim), sin[position_ids].unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class _Rotary:
    def __init__(self, dim, base=10000.0):
        self.dim, self.base = dim, base

    def __call__(self, x, seq_len):
        inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float64, device=x.device) / self.dim))
        ang = torch.outer(torch.arange(max(seq_len, 4096), dtype=torch.float64, device=x.device), inv)
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().to(x.dtype), emb.sin().to(x.dtype)


class _Cache:
    def __init__(self, window_length, codebook):
        self.window_length, self.codebook = window_length, codebook


class _Self:
    def __init__(self, H, D):
        self.head_dim, self.num_heads, self.num_key_value_heads = D, H, H
        self.rotary_emb = _Rotary(D)

    def _type_guard(self, vectors):
        return vectors


class _Logger:
    def warning_once(self, *a, **k):
        pass


def run(B, H, L, D, C, W, dtype=torch.bfloat16, seed=1, reps=5, device="cuda"):
    """Times the reference's host preparation and its fused-kernel wrapper on synthetic inputs and returns the
    tensors it handed to its kernel, so that the caller can run its own kernels on exactly those."""
    assert L % 128 == 0 and C % 128 == 0
    mods = load_modules()
    captured = {}
    fwd = mods["triton_fused_vq_attn"].vq_attn_forward

    def kernel(*args, **kw):
        captured["args"], captured["kw"] = args, kw
        return fwd(*args, **kw)

    ns = dict(torch=torch, math=math, partial=partial, logger=_Logger(), rotate_half=rotate_half,
              apply_rotary_pos_emb=apply_rotary_pos_emb,
              multi_head_single_quantize=mods["mini_vq"].multi_head_single_quantize, VectorQuantizedReRoPECache=_Cache,
              BLOCK_SIZE=128, vq_prefilling_kernel=kernel)
    exec(compile(extract_method("long_prefilling_sort_based_linear"), "attn_vq.py:fast", "exec"), ns)
    fast = ns["long_prefilling_sort_based_linear"]
    g = torch.Generator(device=device).manual_seed(seed)
    q, k, v = (torch.randn(B, H, L, D, generator=g, device=device, dtype=torch.float32).to(dtype) for _ in range(3))
    cb = (torch.randn(H, C, D, generator=g, device=device, dtype=torch.float32) * D ** -0.25).to(dtype)
    pos = torch.arange(L, device=device).unsqueeze(0).expand(B, -1)
    me, cache = _Self(H, D), _Cache(W, cb)

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            r = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, r

    with torch.no_grad():
        out = fast(me, q, k, v, pos, L, cache)                       # warm-up: JIT compilation of both kernels
        total_ms, out = timed(lambda: fast(me, q, k, v, pos, L, cache), max(1, reps // 2))
        args, kw = captured["args"], captured["kw"]
        kernel_ms, o_kernel = timed(lambda: fwd(*args, **kw), reps)
    return dict(total_ms=total_ms, kernel_ms=kernel_ms, prep_ms=total_ms - kernel_ms, out=out, kernel_args=args, kernel_kw=kw,
                inputs=dict(q=q, k=k, v=v, codebook=cb, window=W))
