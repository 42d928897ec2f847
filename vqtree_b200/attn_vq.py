"""Mirror of the reference's ``ops/attn_vq.py`` on the CUDA library: ``BLOCK_SIZE``, ``AttentionMode``,
``VectorQuantizedReRoPECache``, ``LlamaFlashAttention2VectorQuantizedReRoPE`` and ``use_rerope``.

Same names, constructor arguments, ``forward`` / ``_dispatch_attn_impl`` signatures and error behaviour
as the reference (ops/attn_vq.py:23-28, 31-173, 176-248, 482-486).  What differs is underneath: the
rotations, the code assignment, the aggregates and the attention are kernels of ``libvqattn.so``; the
cache keeps a window of the newest keys plus running per-code aggregates, so that generation after a
prefill works (the reference's own cache update is unfinished, ops/attn_vq.py:128-165).

transformers compatibility: releases that still have ``LLAMA_ATTENTION_CLASSES`` (4.36 - 4.47) get the
class installed there, exactly as the reference does; later releases removed that registry and rotate
q/k before any pluggable attention function runs, so there ``use_rerope`` swaps
``modeling_llama.LlamaAttention`` itself for the duration of the context (models built inside it use
the patched class).  ``forward`` accepts both calling conventions (``past_key_value=`` returning three
values, ``past_key_values=`` returning two).
"""
from __future__ import annotations

import math
from contextlib import contextmanager
from enum import Enum
from typing import Any, Dict, Optional, Tuple

import torch

from . import api

BLOCK_SIZE = 128  # ops/attn_vq.py:23 ("MUST MATCH KERNEL")

try:  # the HF pieces are needed for the module class only; the functional entry points work without them
    from transformers.cache_utils import Cache as _HFCache
    from transformers.models.llama import modeling_llama as _modeling_llama
    _LlamaAttention = _modeling_llama.LlamaAttention
except Exception:  # pragma: no cover - transformers missing
    _HFCache = object
    _modeling_llama = None
    _LlamaAttention = torch.nn.Module


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


class VectorQuantizedReRoPECache(_HFCache):
    """The object the reference passes as ``past_key_value`` (ops/attn_vq.py:31-52), with a working update.

    ``codebook`` is [H,C,D] (the reference's single codebook) or [H,M,K,D] (M additive codebooks).
    Per layer the cache holds: a window of the newest keys (rotated and raw) and values, starting at the
    128-block boundary of the next query; counts and fp32 value sums per code of every older key
    (``key_cache`` / ``value_cache`` in the reference's naming, ops/attn_vq.py:143-147) plus a copy of the
    sums in the activation dtype; and the number of tokens seen.
    """

    is_compileable = False

    def __init__(self, window_length: int, codebook: torch.Tensor, sphere: bool = False, *,
                 attention_mode: AttentionMode = AttentionMode.SORT_BASED_LINEAR, rope_base: Optional[float] = None):
        if _HFCache is not object:
            try:
                super().__init__(layers=[])
            except TypeError:  # releases whose Cache.__init__ takes no arguments
                super().__init__()
        assert window_length % BLOCK_SIZE == 0
        self.window_length = window_length
        self.codebook = codebook
        self.codebooks = codebook if codebook.dim() == 4 else codebook[:, None]   # [H,M,K,D]
        assert self.codebook.shape[1] % 128 == 0 or codebook.dim() == 4            # ops/attn_vq.py:45
        assert (self.codebooks.shape[1] * self.codebooks.shape[2]) % BLOCK_SIZE == 0
        self.rotated_codebook = None
        self.sphere = sphere
        self.attention_mode = attention_mode
        self.rope_base = rope_base          # None: taken from the model config by the attention module
        self.seen_tokens = 0                # ops/attn_vq.py:49
        self.states: Dict[int, dict] = {}   # per layer
        self._cb_f32 = None
        self._cb_act: Dict[torch.dtype, torch.Tensor] = {}

    # ---- reference attributes (ops/attn_vq.py:36-40) as views of the per-layer state
    @property
    def key_cache(self):
        return [self.states[i]["cnt"] for i in sorted(self.states)]

    @property
    def value_cache(self):
        return [self.states[i]["vsum32"] for i in sorted(self.states)]

    @property
    def key_buffers(self):
        return [self._window(self.states[i], "win_k1") for i in sorted(self.states)]

    @property
    def value_buffers(self):
        return [self._window(self.states[i], "win_v") for i in sorted(self.states)]

    # ---- HF Cache interface
    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        st = self.states.get(layer_idx or 0)
        return 0 if st is None else st["n"]

    def get_max_length(self) -> Optional[int]:
        return int(1e8)  # "some safe number" (ops/attn_vq.py:85-87)

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return -1

    def get_usable_length(self, new_seq_length: int, layer_idx: Optional[int] = 0) -> int:
        """Cached tokens that a call with ``new_seq_length`` new ones can use (the transformers 4.36 rule the
        reference relies on at ops/attn_vq.py:212)."""
        max_length = self.get_max_length()
        previous = self.get_seq_length(layer_idx)
        if max_length is not None and previous + new_seq_length > max_length:
            return max_length - new_seq_length
        return previous

    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        q_len = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.get_seq_length(layer_idx) + q_len, 0

    @property
    def is_sliding(self):
        return [False] * max(1, len(self.states))

    def __len__(self):
        return len(self.states)

    def reorder_cache(self, beam_idx: torch.LongTensor):  # ops/attn_vq.py:167-173
        for st in self.states.values():
            for name in ("win_k1", "win_k3", "win_v", "cnt", "vsum32", "vsum"):
                if st.get(name) is not None:
                    st[name] = st[name].index_select(0, beam_idx.to(st[name].device))

    # ---- codebook copies the kernels want
    def codebooks_f32(self, device) -> torch.Tensor:
        if self._cb_f32 is None or self._cb_f32.device != torch.device(device):
            self._cb_f32 = self.codebooks.to(device=device, dtype=torch.float32).contiguous()
        return self._cb_f32

    def codebook_act(self, dtype, device) -> torch.Tensor:
        cb = self._cb_act.get(dtype)
        if cb is None or cb.device != torch.device(device):
            H, M, K, D = self.codebooks.shape
            cb = self._cb_act[dtype] = self.codebooks_f32(device).reshape(H, M * K, D).to(dtype).contiguous()
        return cb

    # ---- state
    @staticmethod
    def _window(st, name):
        return st[name][:, :, st["start"]: st["start"] + st["n"] - st["bd"]]

    def update_prefill(self, cumulated_key, cumulated_value, local_key, local_value, layer_idx, num_tokens,
                       cache_kwargs: Optional[Dict[str, Any]] = None):
        """ops/attn_vq.py:89-126: stores what a prefill leaves behind for layer ``layer_idx``.

        cumulated_key [B,Hkv,MK] f32 counts and cumulated_value [B,Hkv,MK,D] f32 value sums of the keys
        before the boundary; local_key (rotated) / local_value [B,Hkv,n_local,D]: the keys from the boundary
        on.  ``cache_kwargs["key_unrotated"]`` carries the raw local keys (scored with the constant-position
        query once they leave the exact window)."""
        if layer_idx in self.states:
            raise RuntimeError("Are you prefilling twice?")  # ops/attn_vq.py:126
        raw = (cache_kwargs or {}).get("key_unrotated")
        assert raw is not None, "cache_kwargs['key_unrotated'] is required"
        B, Hkv, n_local, D = local_key.shape
        dev, dt = local_key.device, local_key.dtype
        cap = 2 * (self.window_length + 2 * BLOCK_SIZE)     # window slides through the buffer; see _make_room
        bufs = [torch.zeros(B, Hkv, cap, D, dtype=dt, device=dev) for _ in range(3)]
        for buf, src in zip(bufs, (local_key, raw, local_value)):
            buf[:, :, :n_local] = src
        vs32 = cumulated_value.float().contiguous()
        self.states[layer_idx] = dict(
            n=num_tokens, bd=num_tokens - n_local, start=0, cap=cap, win_k1=bufs[0], win_k3=bufs[1], win_v=bufs[2],
            cnt=cumulated_key.float().contiguous(), vsum32=vs32, vsum=None if dt == torch.float32 else vs32.to(dt),
            q1=None, q2=None, call=None)
        if layer_idx == 0:
            self.seen_tokens += num_tokens

    def _admit(self, st, dev):
        """Makes room for the token at position ``st["n"]``: when it crosses a 128-block boundary the 128 oldest
        window keys are quantised and folded into the aggregates first.  Returns its buffer row."""
        W = self.window_length
        i = st["n"]
        bd = max(0, (i - W) // BLOCK_SIZE * BLOCK_SIZE)
        moved = False
        if bd > st["bd"]:
            assert bd == st["bd"] + BLOCK_SIZE
            K = self.codebooks.shape[2]
            s0 = st["start"]
            codes = api.assign_codes(st["win_k3"][:, :, s0: s0 + BLOCK_SIZE], self.codebooks_f32(dev))
            api.cache_advance(codes, st["win_v"][:, :, s0: s0 + BLOCK_SIZE], K, st["cnt"], st["vsum32"], st["vsum"])
            st["start"] += BLOCK_SIZE
            st["bd"] = bd
            moved = True
        live = i - st["bd"]
        if st["start"] + live + BLOCK_SIZE + 1 > st["cap"]:
            for name in ("win_k1", "win_k3", "win_v"):      # slide the live window back to the front of its buffer
                buf = st[name]
                buf[:, :, :live] = buf[:, :, st["start"]: st["start"] + live].clone()
            st["start"] = 0
            moved = True
        if moved and st.get("call") is not None:
            s0 = st["start"]
            st["call"].rebind_windows(*(st[n][:, :, s0:] for n in ("win_k1", "win_k3", "win_v")))
        return st["start"] + live

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Appends one new token (HF ``Cache.update`` signature, which is how the reference's ``naive_attn``
        calls it, ops/attn_vq.py:458): ``key_states`` / ``value_states`` [B,Hkv,1,D] are the RAW key and the
        value; ``cache_kwargs`` must hold ``query`` [B,Hq,1,D] (raw) and may hold ``position_ids`` [B,1] and
        ``rope_base``.  When the token crosses a 128-block boundary the 128 oldest window keys are quantised
        and folded into the aggregates first.  Returns the window's rotated keys and values; the rotated
        queries are left in the layer state (``q1``, ``q2``)."""
        st = self.states[layer_idx]
        W = self.window_length
        kw = cache_kwargs or {}
        i = st["n"]                                         # position of the new token
        r = self._admit(st, key_states.device)
        q = kw["query"]
        if st["q1"] is None:
            st["q1"], st["q2"] = (torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(2))
        pos_t = kw.get("position_ids")
        base = kw.get("rope_base") or self.rope_base or 10000.0
        api.decode_append(q, key_states, value_states, i, W + 1, st["q1"], st["q2"], st["win_k1"], st["win_k3"], st["win_v"],
                          r, base=base, positions=pos_t.reshape(-1).to(torch.int64).contiguous() if pos_t is not None else None,
                          n_pos=max(i + 1, W + 2))
        st["n"] = i + 1
        if layer_idx == 0:
            self.seen_tokens += 1
        return self._window(st, "win_k1"), self._window(st, "win_v")

    # ---- persistence
    def state_dict(self) -> Dict[str, Any]:
        """Everything needed to continue generating after a reload (plain tensors and numbers)."""
        layers = {}
        for i, st in self.states.items():
            live = st["n"] - st["bd"]
            layers[i] = dict(n=st["n"], bd=st["bd"], cnt=st["cnt"], vsum32=st["vsum32"],
                             **{k: st[k][:, :, st["start"]: st["start"] + live].contiguous() for k in ("win_k1", "win_k3", "win_v")})
        return dict(window_length=self.window_length, codebook=self.codebook, sphere=self.sphere,
                    attention_mode=self.attention_mode.name, rope_base=self.rope_base, seen_tokens=self.seen_tokens,
                    layers=layers)

    def load_state_dict(self, sd: Dict[str, Any]) -> "VectorQuantizedReRoPECache":
        assert sd["window_length"] == self.window_length, "window length differs from the saved cache"
        self.states = {}
        self.seen_tokens = 0
        for i, ly in sd["layers"].items():
            self.update_prefill(ly["cnt"], ly["vsum32"], ly["win_k1"], ly["win_v"], int(i), ly["n"],
                                {"key_unrotated": ly["win_k3"]})
        self.seen_tokens = sd["seen_tokens"]
        return self

    @classmethod
    def from_state_dict(cls, sd: Dict[str, Any]) -> "VectorQuantizedReRoPECache":
        return cls(sd["window_length"], sd["codebook"], sd["sphere"], attention_mode=AttentionMode[sd["attention_mode"]],
                   rope_base=sd.get("rope_base")).load_state_dict(sd)


# ------------------------------------------------------------------------------------------------------
# Functional entry points: what the module's methods call; usable from any attention module.

def _rope_base(past_key_value, rope_base):
    return rope_base or past_key_value.rope_base or 10000.0


def _store_prefill_state(past_key_value, layer_idx, k1, k3, v, codes, q_len, state=None):
    """Window from the boundary of the NEXT query on, and aggregates of everything older.

    state: (counts, fp32 sums) of the keys before that boundary if the aggregate pass of the prefill already formed
    them; otherwise they are summed here."""
    W = past_key_value.window_length
    H, M, K, D = past_key_value.codebooks.shape
    B, Hkv = k3.shape[0], k3.shape[1]
    dev = k3.device
    bd = max(0, (q_len - W) // BLOCK_SIZE * BLOCK_SIZE)
    if state is not None and state[0] is not None:
        cnt, vs32 = state
    else:
        cnt = torch.zeros(B, Hkv, M * K, dtype=torch.float32, device=dev)
        vs32 = torch.zeros(B, Hkv, M * K, D, dtype=torch.float32, device=dev)
        if bd > 0:
            if codes is None:
                codes = api.assign_codes(k3, past_key_value.codebooks_f32(dev))
            api.cache_advance(codes[:, :, :bd], v[:, :, :bd], K, cnt, vs32, None)
    past_key_value.update_prefill(cnt, vs32, k1[:, :, bd:q_len], v[:, :, bd:q_len], layer_idx, q_len,
                                  {"key_unrotated": k3[:, :, bd:q_len]})


def long_prefilling_sort_based_linear(query_states, key_states, value_states, position_ids, kv_seq_len=None,
                                      past_key_value: VectorQuantizedReRoPECache = None, layer_idx: int = 0,
                                      rope_base: Optional[float] = None, impl: str = "auto"):
    """ops/attn_vq.py:336-443: rotations, code assignment, aggregates, fused attention; fills the cache.

    query_states [B,Hq,L,D], key/value_states [B,Hkv,L,D] (un-rotated; strided views of [B,L,H,D] storage
    are used in place), position_ids [B,L].  Returns [B, L, Hq*D] like the reference (:442) - written by the
    kernel in that layout, no transposing copy."""
    bsz, hq, q_len, d = query_states.shape
    W = past_key_value.window_length
    dev = query_states.device
    n_pos = max(kv_seq_len or q_len, q_len, W + 2)
    q1, q2, k1 = api.rope_qk(query_states, key_states, position_ids, const_pos=W + 1,
                             base=_rope_base(past_key_value, rope_base), n_pos=n_pos, like_input=True)   # :402-407
    out = torch.empty(bsz, q_len, hq, d, dtype=query_states.dtype, device=dev)
    _, st = api.vq_attention_prefill(q1, q2, k1, key_states, value_states, past_key_value.codebooks_f32(dev), W,
                                     scale=1.0 / math.sqrt(d), return_state=True, out=out.transpose(1, 2), impl=impl,
                                     codebook_act=past_key_value.codebook_act(query_states.dtype, dev),
                                     state_blocks=max(0, (q_len - W) // BLOCK_SIZE))
    _store_prefill_state(past_key_value, layer_idx, k1, key_states, value_states, st["codes"], q_len,
                         (st.get("state_cnt"), st.get("state_vsum")))
    return out.flatten(2)


def long_prefilling_slow_reference_impl(query_states, key_states, value_states, position_ids, kv_seq_len=None,
                                        past_key_value: VectorQuantizedReRoPECache = None, layer_idx: int = 0,
                                        rope_base: Optional[float] = None):
    """ops/attn_vq.py:278-334 names a per-query Python loop "only for checking the correctness of linear-time
    prefilling".  Here the cross-check is a second, independent CUDA kernel: fp32 arithmetic, one warp per
    query row, no tensor cores (``impl="simt"``), on the same aggregates."""
    return long_prefilling_sort_based_linear(query_states, key_states, value_states, position_ids, kv_seq_len,
                                             past_key_value, layer_idx, rope_base, impl="simt")


def naive_attn(query_states, key_states, value_states, position_ids, kv_seq_len=None,
               past_key_value: VectorQuantizedReRoPECache = None, layer_idx: int = 0, rope_base: Optional[float] = None):
    """ops/attn_vq.py:445-479: the short-sequence path.  A prefill of at most window + 128 tokens is plain
    causal attention over rotated q / k (what the reference hands to flash-attn, :470-476): the fused kernel
    with q2 = q1, k3 = k1 and a window that covers the whole sequence.  One token on a filled cache is a
    decode step."""
    bsz, hq, q_len, d = query_states.shape
    W = past_key_value.window_length
    dev = query_states.device
    if past_key_value.get_seq_length(layer_idx) > 0:
        return decode_step(query_states, key_states, value_states, position_ids, past_key_value, layer_idx, rope_base)
    n_pos = max(kv_seq_len or q_len, q_len, W + 2)
    q1, _, k1 = api.rope_qk(query_states, key_states, position_ids, base=_rope_base(past_key_value, rope_base),
                            n_pos=n_pos, like_input=True)
    out = torch.empty(bsz, q_len, hq, d, dtype=query_states.dtype, device=dev)
    cover = (q_len + BLOCK_SIZE - 1) // BLOCK_SIZE * BLOCK_SIZE
    api.prefill_from_aggregates(q1, q1, k1, k1, value_states, None, None, None, cover, scale=1.0 / math.sqrt(d),
                                out=out.transpose(1, 2))
    _store_prefill_state(past_key_value, layer_idx, k1, key_states, value_states, None, q_len)
    return out.flatten(2)


def decode_step(query_states, key_states, value_states, position_ids, past_key_value: VectorQuantizedReRoPECache,
                layer_idx: int = 0, rope_base: Optional[float] = None):
    """One generated token (seqlen_q == 1): the decode kernel the reference's README names, on the cache
    this module maintains.  query_states [B,Hq,1,D], key/value_states [B,Hkv,1,D] (un-rotated), position_ids
    [B,1] or None (the cache's own count).  One call into the library, two launches (rotate-and-append,
    attention); two more every 128 tokens when a block leaves the window.  Returns [B, 1, Hq*D]."""
    st = past_key_value.states[layer_idx]
    W = past_key_value.window_length
    bsz, hq, _, d = query_states.shape
    hkv = key_states.shape[1]
    dev = query_states.device
    if st["call"] is None:
        dt = query_states.dtype
        st["q1"], st["q2"] = (torch.empty(bsz, hq, 1, d, dtype=dt, device=dev) for _ in range(2))
        s0 = st["start"]
        st["call"] = api.DecodeStepCall(
            st["q1"], st["q2"], *(st[n][:, :, s0:] for n in ("win_k1", "win_k3", "win_v")),
            past_key_value.codebook_act(dt, dev), st["cnt"], st["vsum"] if st["vsum"] is not None else st["vsum32"],
            api.decode_workspace(bsz, hq, hkv, d, dev), W + 1, _rope_base(past_key_value, rope_base), 1.0 / math.sqrt(d))
    i = st["n"]
    r = past_key_value._admit(st, dev)
    bd = st["bd"]
    pos_t = position_ids.reshape(-1).to(torch.int64).contiguous() if position_ids is not None else None
    out = st["call"](query_states, key_states, value_states, i, r - st["start"], i - bd + 1, max(0, i - W) - bd, bd > 0, pos_t)
    st["n"] = i + 1
    if layer_idx == 0:
        past_key_value.seen_tokens += 1
    return out.reshape(bsz, 1, hq * d)


def dispatch_attn_impl(query_states, key_states, value_states, position_ids, past_key_value: VectorQuantizedReRoPECache,
                       layer_idx: int = 0, rope_base: Optional[float] = None, kv_seq_len: Optional[int] = None):
    """The routing of ops/attn_vq.py:192-196,225-248 for callers without the module class.  Returns [B, q_len, Hq*D]."""
    q_len = query_states.shape[2]
    seen = past_key_value.get_seq_length(layer_idx)
    assert seen == 0 or q_len == 1, "Only support prefilling or generation"  # ops/attn_vq.py:192-196
    inputs = (query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value, layer_idx, rope_base)
    if seen == 0 and q_len > past_key_value.window_length + BLOCK_SIZE:
        if past_key_value.attention_mode == AttentionMode.SORT_BASED_LINEAR:
            return long_prefilling_sort_based_linear(*inputs)
        elif past_key_value.attention_mode == AttentionMode.SLOW_REFERNECE:
            return long_prefilling_slow_reference_impl(*inputs)
        raise KeyError(f"Bad attention mode: {past_key_value.attention_mode}")  # ops/attn_vq.py:246
    return naive_attn(*inputs)


# ------------------------------------------------------------------------------------------------------
# The attention module (ops/attn_vq.py:176-248)

def _config_rope_base(config) -> float:
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and "rope_theta" in rp:
        kind = rp.get("rope_type", "default")
        assert kind in (None, "default"), f"rope_type {kind!r} is not supported by the VQ attention path"
        return float(rp["rope_theta"])
    scaling = getattr(config, "rope_scaling", None)
    assert not scaling or scaling.get("rope_type", scaling.get("type", "default")) == "default", \
        "scaled rotary embeddings are not supported by the VQ attention path"
    return float(getattr(config, "rope_theta", 10000.0))


class LlamaFlashAttention2VectorQuantizedReRoPE(_LlamaAttention):
    """``LlamaAttention`` whose attention is the fused VQ path (ops/attn_vq.py:176-479).

    ``apply_o_proj``: the reference returns the attention output WITHOUT the output projection (the call is
    commented out, ops/attn_vq.py:218) and its self-test compares exactly that; False reproduces it.  Inside a
    full model the projection is wanted: ``use_rerope(o_proj=True)`` turns it on for the models built there.
    """

    apply_o_proj = False

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.LongTensor] = None,
                position_ids: Optional[torch.LongTensor] = None, past_key_value=None, output_attentions: bool = False,
                use_cache: bool = False, **kwargs):
        new_api = past_key_value is None and "past_key_values" in kwargs   # transformers >= 4.48 calling convention
        if past_key_value is None:
            past_key_value = kwargs.get("past_key_values")
        bsz, q_len, _ = hidden_states.size()

        assert isinstance(past_key_value, VectorQuantizedReRoPECache), "VQReRoPECache is required"
        assert (
            past_key_value.get_seq_length(self.layer_idx) == 0 or q_len == 1
        ), "Only support prefilling or generation"
        assert not output_attentions, "Not implemented"
        assert not self.training, "Not implemented"
        assert not past_key_value.sphere, "Not implemented"

        num_heads = self.config.num_attention_heads
        num_kv_heads = self.config.num_key_value_heads
        # [B,L,H,D] storage viewed as [B,H,L,D] (ops/attn_vq.py:207-209); the kernels read the views in place
        query_states = self.q_proj(hidden_states).view(bsz, q_len, num_heads, self.head_dim).transpose(1, 2)
        key_states = self.k_proj(hidden_states).view(bsz, q_len, num_kv_heads, self.head_dim).transpose(1, 2)
        value_states = self.v_proj(hidden_states).view(bsz, q_len, num_kv_heads, self.head_dim).transpose(1, 2)

        kv_seq_len = key_states.shape[-2]
        kv_seq_len += past_key_value.get_usable_length(kv_seq_len, self.layer_idx)

        attn_output = self._dispatch_attn_impl(query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value)
        if self.apply_o_proj:
            attn_output = self.o_proj(attn_output)
        if new_api:
            return attn_output, None
        return attn_output, None, past_key_value

    def _rope_base(self) -> float:
        return _config_rope_base(self.config)

    def _dispatch_attn_impl(self, query_states, key_states, value_states, position_ids, kv_seq_len,
                            past_key_value: VectorQuantizedReRoPECache):
        is_prefilling = past_key_value.get_seq_length(self.layer_idx) == 0
        is_prefilling_with_memory = is_prefilling and query_states.shape[2] > past_key_value.window_length + BLOCK_SIZE
        inputs = (query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value)
        if is_prefilling_with_memory:
            if past_key_value.attention_mode == AttentionMode.SORT_BASED_LINEAR:
                return self.long_prefilling_sort_based_linear(*inputs)
            elif past_key_value.attention_mode == AttentionMode.SLOW_REFERNECE:
                return self.long_prefilling_slow_reference_impl(*inputs)
            raise KeyError(f"Bad attention mode: {past_key_value.attention_mode}")
        else:
            return self.naive_attn(query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value)

    def _type_guard(self, vectors):
        """ops/attn_vq.py:250-276: fp32 activations are cast to the projection weights' dtype."""
        single = isinstance(vectors, torch.Tensor)
        vectors = [vectors] if single else list(vectors)
        if vectors[0].dtype == torch.float32 and self.q_proj.weight.dtype != torch.float32:
            target = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else self.q_proj.weight.dtype
            vectors = [v.to(target) for v in vectors]
        return vectors[0] if single else vectors

    def long_prefilling_sort_based_linear(self, query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value):
        query_states, key_states, value_states = self._type_guard((query_states, key_states, value_states))
        return long_prefilling_sort_based_linear(query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value,
                                                 self.layer_idx, self._rope_base())

    def long_prefilling_slow_reference_impl(self, query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value):
        query_states, key_states, value_states = self._type_guard((query_states, key_states, value_states))
        return long_prefilling_slow_reference_impl(query_states, key_states, value_states, position_ids, kv_seq_len,
                                                   past_key_value, self.layer_idx, self._rope_base())

    def naive_attn(self, query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value):
        query_states, key_states, value_states = self._type_guard((query_states, key_states, value_states))
        return naive_attn(query_states, key_states, value_states, position_ids, kv_seq_len, past_key_value, self.layer_idx,
                          self._rope_base())


@contextmanager
def use_rerope(o_proj: bool = False):
    """ops/attn_vq.py:482-486: models built inside the context get the VQ attention class.

    With a transformers release that has ``LLAMA_ATTENTION_CLASSES`` the "flash_attention_2" entry is swapped
    and restored, as in the reference; otherwise ``modeling_llama.LlamaAttention`` is."""
    assert _modeling_llama is not None, "transformers is required for use_rerope()"
    cls = LlamaFlashAttention2VectorQuantizedReRoPE
    if o_proj:
        cls = type(cls.__name__, (cls,), {"apply_o_proj": True})
    registry = getattr(_modeling_llama, "LLAMA_ATTENTION_CLASSES", None)
    if registry is not None:
        saved = registry["flash_attention_2"]
        registry["flash_attention_2"] = cls
        try:
            yield
        finally:
            registry["flash_attention_2"] = saved
    else:
        saved = _modeling_llama.LlamaAttention
        _modeling_llama.LlamaAttention = cls
        try:
            yield
        finally:
            _modeling_llama.LlamaAttention = saved
