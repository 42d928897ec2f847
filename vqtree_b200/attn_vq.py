"""Mirror of the reference's ``ops/attn_vq.py`` for the VQ path: block size, attention modes, the
cache object and the prefill / decode dispatch, on the CUDA library.

The HF ``LlamaAttention`` subclass of the reference (ops/attn_vq.py:176-248) depends on a
transformers API (``LlamaFlashAttention2``, ``LLAMA_ATTENTION_CLASSES``) that newer releases removed;
the functions here take the projected ``[B,H,L,D]`` states that class hands to its dispatch
(``_dispatch_attn_impl``, :225-248) and can be called from any attention module.
"""
from __future__ import annotations

import math
from enum import Enum
from typing import Optional

import torch

from . import api

BLOCK_SIZE = 128  # ops/attn_vq.py:23


class AttentionMode(Enum):  # ops/attn_vq.py:26-28 (the spelling of the first member is the reference's)
    SLOW_REFERNECE = 0
    SORT_BASED_LINEAR = 1


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_cos_sin(n_pos: int, dim: int, device, base: float = 10000.0):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim))
    ang = torch.outer(torch.arange(n_pos, dtype=torch.float64, device=device), inv)
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().float(), ang.sin().float()


class VectorQuantizedReRoPECache:
    """State the reference passes as ``past_key_value`` (ops/attn_vq.py:31-52) plus what decode needs.

    ``codebook`` is [H,C,D] (the reference's single codebook) or [H,M,K,D].  After a prefill the cache
    holds, per layer, the newest window of rotated keys, un-rotated keys and values, the running
    counts and fp32 value sums of everything older, and the number of tokens seen.
    """

    def __init__(self, window_length: int, codebook: torch.Tensor, sphere: bool = False, *,
                 attention_mode: AttentionMode = AttentionMode.SORT_BASED_LINEAR):
        assert window_length % BLOCK_SIZE == 0
        assert not sphere, "Not implemented"  # ops/attn_vq.py:198
        self.window_length = window_length
        self.codebook = codebook if codebook.dim() == 4 else codebook[:, None]
        assert (self.codebook.shape[1] * self.codebook.shape[2]) % BLOCK_SIZE == 0  # ops/attn_vq.py:45
        self.sphere = sphere
        self.attention_mode = attention_mode
        self.layers = {}
        self.seen_tokens = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        st = self.layers.get(layer_idx)
        return 0 if st is None else st["n"]


def long_prefilling_sort_based_linear(query_states, key_states, value_states, position_ids,
                                      past_key_value: VectorQuantizedReRoPECache, layer_idx: int = 0,
                                      rope_base: float = 10000.0):
    """ops/attn_vq.py:336-443: RoPE / ReRoPE rotation, code assignment, aggregates, fused attention.

    query_states [B,Hq,L,D], key/value_states [B,Hkv,L,D] (un-rotated), position_ids [B,L].
    Returns [B, L, Hq*D] like the reference (:442).
    """
    bsz, hq, q_len, d = query_states.shape
    W = past_key_value.window_length
    n_pos = max(q_len, W + 2)
    q1, q2 = api.rope(query_states, position_ids, const_pos=W + 1, base=rope_base, n_pos=n_pos)  # :402-407
    k1, _ = api.rope(key_states, position_ids, base=rope_base, n_pos=n_pos)
    cb = past_key_value.codebook.float().contiguous()
    out, st = api.vq_attention_prefill(q1, q2, k1, key_states.contiguous(), value_states.contiguous(), cb, W,
                                       scale=1.0 / math.sqrt(d), return_state=True)
    past_key_value.layers[layer_idx] = dict(n=q_len, k1=k1, k3=key_states, v=value_states, codes=st["codes"])
    if layer_idx == 0:
        past_key_value.seen_tokens += q_len
    return out.transpose(1, 2).contiguous().flatten(2)


def _decode_state(cache: VectorQuantizedReRoPECache, layer_idx: int):
    """Turns the state a prefill left (all keys) into the decode form: a window of the newest keys from the
    boundary on, and the aggregates (counts, fp32 value sums + their activation-dtype copy) of everything older."""
    st = cache.layers[layer_idx]
    if "win_k1" in st:
        return st
    W = cache.window_length
    n = st["n"]
    k1, k3, v, codes = st["k1"], st["k3"], st["v"], st["codes"]
    B, Hkv, _, D = k3.shape
    _, M, K, _ = cache.codebook.shape
    dev, dt = k3.device, k3.dtype
    bd = max(0, (n - W) // BLOCK_SIZE * BLOCK_SIZE)   # boundary of the NEXT query (position n)
    nwin = W + 2 * BLOCK_SIZE                          # rows [bd, i] never exceed W + 128; one block of slack
    win = lambda t: torch.zeros(B, Hkv, nwin, D, dtype=dt, device=dev)
    st.update(win_k1=win(k1), win_k3=win(k3), win_v=win(v), bd=bd,
              cnt=torch.zeros(B, Hkv, M * K, dtype=torch.float32, device=dev),
              vsum32=torch.zeros(B, Hkv, M * K, D, dtype=torch.float32, device=dev),
              vsum=torch.zeros(B, Hkv, M * K, D, dtype=dt, device=dev) if dt != torch.float32 else None,
              cb_act=cache.codebook.reshape(Hkv, M * K, D).to(dt).contiguous())
    for name, src in (("win_k1", k1), ("win_k3", k3), ("win_v", v)):
        st[name][:, :, : n - bd] = src[:, :, bd:n]
    if bd > 0:
        if codes is None:
            codes = api.assign_codes(k3.contiguous(), cache.codebook.float().contiguous())
        api.cache_advance(codes[:, :, :bd].contiguous(), v[:, :, :bd].contiguous(), K, st["cnt"], st["vsum32"], st["vsum"])
    for name in ("k1", "k3", "v", "codes"):
        st.pop(name)
    return st


def decode_step(query_states, key_states, value_states, position_ids, past_key_value: VectorQuantizedReRoPECache,
                layer_idx: int = 0, rope_base: float = 10000.0):
    """One generated token (seqlen_q == 1): stands in for the reference's unfinished cache update
    (ops/attn_vq.py:128-165) and the decode kernel its README names.

    query_states [B,Hq,1,D], key/value_states [B,Hkv,1,D] (un-rotated), position_ids [B,1] (all equal to the number
    of tokens seen).  The new key joins the window; when the boundary moves (every 128 tokens) the 128 oldest
    window keys are quantised and folded into the aggregates.  Returns [B, 1, Hq*D].
    """
    st = _decode_state(past_key_value, layer_idx)
    W = past_key_value.window_length
    i = st["n"]                                        # position of the new token
    assert int(position_ids.reshape(-1)[0]) == i, "decode_step expects the next position"
    bsz, hq, _, d = query_states.shape
    _, M, K, _ = past_key_value.codebook.shape
    n_pos = max(i + 1, W + 2)
    q1, q2 = api.rope(query_states, position_ids, const_pos=W + 1, base=rope_base, n_pos=n_pos)
    k1_new, _ = api.rope(key_states, position_ids, base=rope_base, n_pos=n_pos)
    q1, q2 = q1[:, :, 0], q2[:, :, 0]
    bd = max(0, (i - W) // BLOCK_SIZE * BLOCK_SIZE)
    if bd > st["bd"]:
        # the boundary moved by one block: its keys leave the window for the aggregates
        assert bd == st["bd"] + BLOCK_SIZE
        old_k3 = st["win_k3"][:, :, :BLOCK_SIZE].contiguous()
        codes = api.assign_codes(old_k3, past_key_value.codebook.float().contiguous())
        api.cache_advance(codes, st["win_v"][:, :, :BLOCK_SIZE].contiguous(), K, st["cnt"], st["vsum32"], st["vsum"])
        for name in ("win_k1", "win_k3", "win_v"):
            st[name] = torch.roll(st[name], -BLOCK_SIZE, dims=2)
        st["bd"] = bd
    r = i - bd                                         # window row of the new key
    st["win_k1"][:, :, r] = k1_new[:, :, 0]
    st["win_k3"][:, :, r] = key_states[:, :, 0]
    st["win_v"][:, :, r] = value_states[:, :, 0]
    far = bd > 0
    vs = st["vsum"] if st["vsum"] is not None else st["vsum32"]
    out = api.vq_attention_decode(q1.contiguous(), q2.contiguous(), st["win_k1"], st["win_k3"], st["win_v"],
                                  st["cb_act"] if far else None, st["cnt"] if far else None, vs if far else None,
                                  n_valid=r + 1, n_bd=max(0, i - W) - bd, scale=1.0 / math.sqrt(d))
    st["n"] = i + 1
    if layer_idx == 0:
        past_key_value.seen_tokens += 1
    return out.reshape(bsz, 1, hq * d)


def dispatch_attn_impl(query_states, key_states, value_states, position_ids, past_key_value: VectorQuantizedReRoPECache,
                       layer_idx: int = 0, rope_base: float = 10000.0):
    """The routing of ops/attn_vq.py:192-196,225-248 over this module's entry points.

    An empty cache means prefilling (any length: without far keys the fused kernel computes the exact window
    attention the reference hands to its short-sequence path); a filled cache accepts one token at a time.
    Returns [B, q_len, Hq*D].
    """
    q_len = query_states.shape[2]
    seen = past_key_value.get_seq_length(layer_idx)
    assert seen == 0 or q_len == 1, "Only support prefilling or generation"  # ops/attn_vq.py:192-196
    if seen == 0:
        if past_key_value.attention_mode not in (AttentionMode.SORT_BASED_LINEAR, AttentionMode.SLOW_REFERNECE):
            raise KeyError(f"Bad attention mode: {past_key_value.attention_mode}")  # ops/attn_vq.py:246
        # SLOW_REFERNECE names the reference's per-query loop; its results are what the fused path is tested against
        return long_prefilling_sort_based_linear(query_states, key_states, value_states, position_ids, past_key_value,
                                                 layer_idx, rope_base)
    return decode_step(query_states, key_states, value_states, position_ids, past_key_value, layer_idx, rope_base)
