"""Generate the golden vectors in this folder by running the reference's own code.

Run once, in a container that has the reference checkout:

    TRITON_INTERPRET=1 python tests/golden/gen_golden.py --ref <reference checkout>

Nothing from the reference is copied: its files are loaded (or, for two methods of a class
that cannot be imported with the installed transformers, parsed and executed) where they lie,
and only seeded inputs and the outputs they produce are stored, as small ``.npz`` files.

What is executed, and what it pins:

* ``ops/mini_vq.py`` ``multi_head_single_quantize`` (imported by path)  -> ``assign_*.npz``
* ``ops/attn_vq.py`` ``long_prefilling_slow_reference_impl`` (method source parsed with ``ast``
  and executed against a stand-in ``self``; rotary helpers follow the HF Llama half-split
  convention the method expects)                                           -> ``naive_*.npz``
* ``ops/attn_vq.py`` ``long_prefilling_sort_based_linear`` (same technique): the host
  preparation of counts, sorted value prefix sums and row indices; its call of the fused kernel
  is served by the reference's two Triton kernels ``_fwd_kernel`` (local ReRoPE window) and
  ``_vq_fwd_kernel`` (far part) run by the Triton interpreter on CPU in fp32, launched with the
  argument order of the reference's own call sites, and merged with the log-sum-exp formula
  of the cascade merge the reference calls                                  -> ``fast_*.npz``

The test-suite checks the CPU oracle against these files; they are never regenerated at test
time and the reference is not needed to run the tests.
"""
from __future__ import annotations

import argparse
import ast
import importlib.util
import math
import os
import sys
import textwrap
import types
from functools import partial
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_ref_modules(ref: Path):
    """Load the three hot-path files by path, bypassing ops/__init__.py."""
    pkg = types.ModuleType("ops")
    pkg.__path__ = [str(ref / "ops")]
    sys.modules["ops"] = pkg
    mods = {}
    for name in ("mini_vq", "triton_fused_local_attn_rerope", "triton_fused_vq_attn"):
        spec = importlib.util.spec_from_file_location(f"ops.{name}", ref / "ops" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"ops.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def extract_method(ref: Path, cls: str, name: str):
    """Return the source of ``cls.name`` from ops/attn_vq.py as a plain function definition."""
    src = (ref / "ops" / "attn_vq.py").read_text()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == cls:
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and item.name == name:
                    return textwrap.dedent(ast.get_source_segment(src, item))
    raise KeyError(name)


# ---- stand-ins for the transformers helpers the two methods call (HF Llama, ~4.37 API) ----

def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids, unsqueeze_dim=1):
    cos = cos[position_ids].unsqueeze(unsqueeze_dim)
    sin = sin[position_ids].unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class _Rotary:
    def __init__(self, dim, base=10000.0):
        self.inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))

    def __call__(self, x, seq_len):
        # tables long enough for position window+1 as well
        t = torch.arange(max(seq_len, 4096), dtype=torch.float64)
        freqs = torch.outer(t, self.inv_freq)
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(x.dtype), emb.sin().to(x.dtype)


class _Logger:
    def warning_once(self, *a, **k):
        pass


class _Cache:
    def __init__(self, window_length, codebook):
        self.window_length = window_length
        self.codebook = codebook


class _Self:
    def __init__(self, H, D):
        self.head_dim = D
        self.num_heads = H
        self.num_key_value_heads = H
        self.rotary_emb = _Rotary(D)

    def _type_guard(self, vectors):
        return vectors


def interpreted_fused_kernel(mods, captured):
    """Stand-in for the fused kernel entry: runs the reference's two Triton kernels on CPU."""
    local = mods["triton_fused_local_attn_rerope"]
    far = mods["triton_fused_vq_attn"]

    def run(q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi, window_size, softmax_scale=None):
        q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi = [
            x if x.stride(-1) == 1 else x.contiguous() for x in (q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi)
        ]
        B, H, L, D = q1.shape
        scale = softmax_scale or 1.0 / math.sqrt(D)
        # local kernel: inputs viewed as [B, L, H, D]; call-site order of
        # ops/triton_fused_local_attn_rerope.py:258-281
        tq1, tq2, tk1, tk3, tv = (x.transpose(1, 2) for x in (q1, q2, k1, k3, v))
        o1 = torch.empty_like(tq1, memory_format=torch.contiguous_format)
        l1 = torch.empty((B, H, L), dtype=torch.float32)
        grid = (-(-L // 128), B * H)
        local._fwd_kernel[grid](
            tq1, tq2, tk1, tk3, tv, o1, l1, scale,
            tq1.stride(0), tq1.stride(2), tq1.stride(1),
            tk1.stride(0), tk1.stride(2), tk1.stride(1),
            tv.stride(0), tv.stride(2), tv.stride(1),
            o1.stride(0), o1.stride(2), o1.stride(1),
            H, L, L, L // 32, L // 32, window_size, D,
            BLOCK_M=128, BLOCK_N=128, WRITE_LSE=True, num_warps=4, num_stages=1,
        )
        o1 = o1.transpose(1, 2)  # [B,H,L,D]
        # far kernel: call-site order of ops/triton_fused_vq_attn.py:223-245
        o2 = torch.zeros_like(q1, memory_format=torch.contiguous_format)
        l2 = torch.full((B, H, L), float("-inf"), dtype=torch.float32)
        nblk = -(-(L - window_size - 128) // 128)
        if nblk > 0:
            far._vq_fwd_kernel[(nblk, B * H)](
                q2, k_vq, k_vq_cnt, v_vq, vi, o2, l2, scale,
                *q2.stride()[:-1], *k_vq.stride()[:-1], *k_vq_cnt.stride()[:-1], *v_vq.stride()[:-1],
                *vi.stride()[:-1], *o2.stride()[:-1],
                H, L, k_vq.shape[1], L // 32, window_size, D,
                BLOCK_M=128, BLOCK_N=128, WRITE_LSE=True, num_warps=4, num_stages=1,
            )
        # cascade merge in base 2 (what the merge at ops/triton_fused_vq_attn.py:246-250 computes)
        mx = torch.maximum(l1, l2)
        w1, w2 = torch.exp2(l1 - mx), torch.exp2(l2 - mx)
        merged = (o1 * w1[..., None] + o2 * w2[..., None]) / (w1 + w2)[..., None]
        captured.update(k_vq_cnt=k_vq_cnt.clone(), v_vq=v_vq.clone(), vi=vi.clone(), o_local=o1.clone(),
                        lse_local=l1.clone(), o_far=o2.clone(), lse_far=l2.clone(), q2=q2.clone(), k1=k1.clone(),
                        q1=q1.clone())
        return merged

    return run


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    ref = Path(args.ref)
    mods = load_ref_modules(ref)
    mini_vq = mods["mini_vq"]

    # ---------------- assignment ----------------
    for tag, (B, H, L, D, C, seed) in {"a": (2, 2, 384, 64, 128, 100), "b": (1, 3, 256, 128, 256, 101)}.items():
        g = torch.Generator().manual_seed(seed)
        k = torch.randn(B, H, L, D, generator=g)
        cb = torch.randn(H, C, D, generator=g) * (D ** -0.25)
        quant, ids, onehot = mini_vq.multi_head_single_quantize(k, cb)
        np.savez_compressed(HERE / f"assign_{tag}.npz", k=k.numpy(), codebook=cb.numpy(), ids=ids.numpy().astype(np.int32),
                            quantized_head=quant[:, :, :8].numpy())
        print("assign", tag, ids.shape, int(onehot.sum()))

    # ---------------- naive loop and fast path ----------------
    slow_src = extract_method(ref, "LlamaFlashAttention2VectorQuantizedReRoPE", "long_prefilling_slow_reference_impl")
    fast_src = extract_method(ref, "LlamaFlashAttention2VectorQuantizedReRoPE", "long_prefilling_sort_based_linear")
    captured = {}
    ns = dict(torch=torch, math=math, partial=partial, logger=_Logger(), rotate_half=rotate_half,
              apply_rotary_pos_emb=apply_rotary_pos_emb, multi_head_single_quantize=mini_vq.multi_head_single_quantize,
              VectorQuantizedReRoPECache=_Cache, BLOCK_SIZE=128,
              vq_prefilling_kernel=interpreted_fused_kernel(mods, captured))
    exec(compile(slow_src, "attn_vq.py:slow", "exec"), ns)
    exec(compile(fast_src, "attn_vq.py:fast", "exec"), ns)
    slow, fast = ns["long_prefilling_slow_reference_impl"], ns["long_prefilling_sort_based_linear"]

    cases = {
        # the reference self-test's shape (ops/attn_vq.py:534-556): LEN 511, window 256, codebook 128 x 64
        "selftest": dict(B=1, H=2, L=511, D=64, C=128, W=256, seed=200),
        "w128": dict(B=1, H=2, L=640, D=64, C=128, W=128, seed=201),
    }
    for tag, c in cases.items():
        B, H, L, D, C, W = c["B"], c["H"], c["L"], c["D"], c["C"], c["W"]
        g = torch.Generator().manual_seed(c["seed"])
        q = torch.randn(B, H, L, D, generator=g)
        k = torch.randn(B, H, L, D, generator=g)
        v = torch.randn(B, H, L, D, generator=g)
        cb = torch.randn(H, C, D, generator=g) * (D ** -0.25)
        pos = torch.arange(L).unsqueeze(0).expand(B, -1)
        me = _Self(H, D)
        cache = _Cache(W, cb)
        with torch.no_grad():
            o_slow = slow(me, q, k, v, pos, L, cache)  # [B, L, H*D]
        o_slow = o_slow.view(B, L, H, D).transpose(1, 2).contiguous()
        np.savez_compressed(HERE / f"naive_{tag}.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), codebook=cb.numpy(),
                            window=W, out=o_slow.numpy())
        print("naive", tag, o_slow.shape)
        if L % 128 == 0:
            captured.clear()
            with torch.no_grad():
                o_fast = fast(me, q, k, v, pos, L, cache)
            o_fast = o_fast.view(B, L, H, D).transpose(1, 2).contiguous()
            err = (o_fast - o_slow).abs().max().item()
            print("fast", tag, "max|fast-slow| =", err)
            np.savez_compressed(
                HERE / f"fast_{tag}.npz", out=o_fast.numpy(), k_vq_cnt=captured["k_vq_cnt"].numpy().astype(np.int32),
                v_vq=captured["v_vq"].numpy(), vi=captured["vi"].numpy().astype(np.int32),
                o_local=captured["o_local"].numpy(), lse_local=captured["lse_local"].numpy(),
                o_far=captured["o_far"].numpy(), lse_far=captured["lse_far"].numpy(),
                q1=captured["q1"].numpy(), q2=captured["q2"].numpy(), k1=captured["k1"].numpy())


if __name__ == "__main__":
    main()
