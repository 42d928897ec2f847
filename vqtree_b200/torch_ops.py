"""``torch.ops.vqattn.*``: the PyTorch C++ extension over the library's C ABI.

``csrc/torch_ext.cpp`` registers the entry points of ``include/vqattn.h`` with PyTorch's dispatcher (CUDA
backend only - a CPU tensor finds no kernel and raises), each as an out-variant that writes into tensors the
caller passes: a C++ device guard, PyTorch's current stream, ``TORCH_CHECK`` errors.  The same kernels as the
ctypes layer (``native.py`` / ``api.py``) run; this binding is for callers that want dispatcher operators
(C++ callers, ``torch.compile`` graphs, TorchScript-free export) instead of a ctypes stub.

    from vqtree_b200 import torch_ops
    ops = torch_ops.load()                     # torch.ops.vqattn
    ops.prefill(q1, q2, k1, k3, v, cb_act, cnt, vsum, window, 0.0, 0, out, None, None)

Operators (argument meaning as in ``include/vqattn.h``; trailing ``status_word`` is the optional device int32
that kernels raise on an expired bounded wait or a bad code):
    assign_codes(k, codebooks, bias?, codes!, workspace?, status_word?)
    build_aggregates(codes, v, K, cnt!, vsum!, state_cnt!?, state_vsum!?, state_blocks, workspace?, status_word?)
    prefill(q1, q2, k1, k3, v, codebook?, cnt?, vsum?, window, scale, impl, out!, lse2!?, status_word?)
    decode(q1, q2, k1_win, k3_win, v_win, codebook?, cnt?, vsum?, n_valid, n_bd, scale, workspace!, out!, status_word?)
    cache_advance(codes, v_new, K, cnt!, vsum_f32!, vsum_act!?, status_word?)
    abi_version(), assign_workspace_bytes(...), aggregates_workspace_bytes(...), decode_workspace_bytes(...)
"""
from __future__ import annotations

from pathlib import Path

import torch

from . import native  # loads libvqattn.so first and fails loudly when it is missing

LIB = Path(__file__).resolve().parent / "lib" / "libvqattn_torch.so"
_MUTATING = ("assign_codes", "build_aggregates", "prefill", "decode", "cache_advance")
_loaded = False


def load():
    """Loads the extension (once) and returns ``torch.ops.vqattn``."""
    global _loaded
    if not _loaded:
        if not LIB.exists():
            raise ImportError(f"{LIB} is missing: run `python -m vqtree_b200.build` (g++ against the installed torch)")
        torch.ops.load_library(str(LIB))
        if int(torch.ops.vqattn.abi_version()) != int(native.lib.vqattn_version()):
            raise ImportError("libvqattn_torch.so was built against another libvqattn.so: rebuild both")
        # shape propagation for tracing: the operators return nothing and only write into their arguments
        for name in _MUTATING:
            torch.library.register_fake(f"vqattn::{name}")(_nothing)
        _loaded = True
    return torch.ops.vqattn


def _nothing(*args, **kwargs):
    return None
