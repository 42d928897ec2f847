"""Codebook files and cache files.

The reference trains its additive quantizers offline and pickles the result as a dict
``{(layer_idx, kv_head_idx): codebooks}`` where ``codebooks`` is what faiss'
``get_additive_quantizer_codebooks`` returns: a list of M float32 arrays ``[2**bits, D]``
(build_quantizer/120_build_additive_quantizer.py:33-35,51,60-66; the sphere variant,
build_quantizer/121_build_sphere_additive_quantizer.py, writes the same structure).  Nothing in the
reference's ``ops/`` reads that file yet; ``load_codebooks`` does, and returns what
``VectorQuantizedReRoPECache`` takes per layer.  ``save_cache`` / ``load_cache`` persist a cache's state
(``VectorQuantizedReRoPECache.state_dict``) with ``torch.save``.
"""
from __future__ import annotations

import io
import pickle
from pathlib import Path
from typing import Dict, Union

import numpy as np
import torch


class _ArraysOnly(pickle.Unpickler):
    """Unpickler that resolves numpy array reconstruction only: a codebook file holds nothing else."""

    _ALLOWED = {
        ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct"),
        ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
        ("numpy", "ndarray"), ("numpy", "dtype"),
        ("numpy.core.numeric", "_frombuffer"), ("numpy._core.numeric", "_frombuffer"),
    }

    def find_class(self, module, name):
        if (module, name) in self._ALLOWED:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"codebook files may only contain numpy arrays, found {module}.{name}")


def save_codebooks(codebooks: Dict[int, Union[torch.Tensor, np.ndarray]], path) -> None:
    """Writes ``{layer: [Hkv, M, K, D]}`` in the reference's pickle layout ``{(layer, head): [M arrays [K, D]]}``."""
    out = {}
    for layer, cb in codebooks.items():
        cb = cb.detach().cpu().numpy() if isinstance(cb, torch.Tensor) else np.asarray(cb)
        assert cb.ndim == 4, "expected [Hkv, M, K, D]"
        for h in range(cb.shape[0]):
            out[(int(layer), h)] = [np.ascontiguousarray(cb[h, m], dtype=np.float32) for m in range(cb.shape[1])]
    with open(path, "wb") as f:
        pickle.dump(out, f)


def load_codebooks(path, device="cpu") -> Dict[int, torch.Tensor]:
    """Reads a codebook pickle of the reference's layout -> ``{layer: tensor [Hkv, M, K, D] float32}``.

    Every (layer, head) of a layer must be present with the same M, K and D; a missing head or a ragged
    shape raises ``ValueError`` naming it."""
    data = Path(path).read_bytes()
    raw = _ArraysOnly(io.BytesIO(data)).load()
    if not isinstance(raw, dict) or not raw:
        raise ValueError("not a codebook file: expected a non-empty dict {(layer, head): codebooks}")
    by_layer: Dict[int, Dict[int, np.ndarray]] = {}
    for key, books in raw.items():
        if not (isinstance(key, tuple) and len(key) == 2):
            raise ValueError(f"bad key {key!r}: expected (layer, head)")
        layer, head = int(key[0]), int(key[1])
        arr = np.stack([np.asarray(b, dtype=np.float32) for b in books]) if isinstance(books, (list, tuple)) else \
            np.asarray(books, dtype=np.float32)
        if arr.ndim == 2:            # a single codebook [K, D]
            arr = arr[None]
        if arr.ndim != 3:
            raise ValueError(f"codebooks of {key}: expected M arrays [K, D], got shape {arr.shape}")
        by_layer.setdefault(layer, {})[head] = arr
    out = {}
    for layer, heads in sorted(by_layer.items()):
        n = max(heads) + 1
        missing = [h for h in range(n) if h not in heads]
        if missing:
            raise ValueError(f"layer {layer}: heads {missing} are missing")
        shapes = {heads[h].shape for h in range(n)}
        if len(shapes) != 1:
            raise ValueError(f"layer {layer}: heads have different codebook shapes {sorted(shapes)}")
        out[layer] = torch.from_numpy(np.stack([heads[h] for h in range(n)])).to(device)
    return out


def save_cache(cache, path) -> None:
    """``torch.save`` of ``cache.state_dict()`` with every tensor moved to the host."""
    def host(x):
        if isinstance(x, torch.Tensor):
            return x.detach().cpu()
        if isinstance(x, dict):
            return {k: host(v) for k, v in x.items()}
        return x
    torch.save(host(cache.state_dict()), path)


def load_cache(path, device="cuda"):
    """Rebuilds a ``VectorQuantizedReRoPECache`` saved by ``save_cache`` on ``device``; generation continues
    from it with the same results as from the original."""
    from .attn_vq import VectorQuantizedReRoPECache
    sd = torch.load(path, map_location=device, weights_only=True)
    return VectorQuantizedReRoPECache.from_state_dict(sd)
