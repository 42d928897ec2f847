"""Scenarios for the attention module and its cache, shared by the CPU suite (kernels replaced by the test
double in tests/fake_backend.py) and the GPU suite (real kernels): the same assertions either way."""
from __future__ import annotations

import numpy as np
import torch

from oracle import vq_oracle as vo


def _f(t):
    return t.detach().float().cpu().numpy()


def oracle_rows(q, k, v, cb, W, dtype, base=10000.0, rows=None):
    """Naive-oracle output [B, L, Hq*D] from RAW q/k/v [B,H,L,D] (already rounded to ``dtype``): rotations in
    fp32 rounded to ``dtype``, codes from the raw keys, codebook rounded to ``dtype`` for the far scores."""
    L, D = q.shape[2], q.shape[3]
    cos, sin = vo.rope_tables(max(L, W + 2), D, base)
    rd = lambda a: _f(torch.from_numpy(np.ascontiguousarray(a)).to(dtype))
    pos = np.arange(L)
    qn, kn, vn = _f(q), _f(k), _f(v)
    q1, k1 = rd(vo.apply_rope(qn, cos, sin, pos)), rd(vo.apply_rope(kn, cos, sin, pos))
    q2 = rd(vo.apply_rope(qn, cos, sin, np.full(L, W + 1)))
    cbn = _f(cb) if cb.dim() == 4 else _f(cb)[:, None]
    codes = vo.assign_codes(kn, cbn)
    out = vo.attn_naive(q1, q2, k1, kn, vn, rd(cbn) if dtype != torch.float32 else cbn, codes, W, rows=rows)
    B, Hq = q.shape[0], q.shape[1]
    return out.transpose(0, 2, 1, 3).reshape(B, L, Hq * D)


def make_module(dtype, device, hidden=128, heads=2, kv_heads=2, seed=0):
    """The reference's self-test module (ops/attn_vq.py:537-540): LlamaConfig(hidden_size=128, 2 heads)."""
    from transformers.models.llama import LlamaConfig
    from vqtree_b200.attn_vq import LlamaFlashAttention2VectorQuantizedReRoPE
    torch.manual_seed(seed)
    config = LlamaConfig(hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads)
    module = LlamaFlashAttention2VectorQuantizedReRoPE(config, layer_idx=0).to(dtype).to(device)
    module.eval()
    return module


def project(module, x):
    """q, k, v [B,H,L,D] exactly as the module computes them."""
    B, L, _ = x.shape
    D = module.head_dim
    hq, hkv = module.config.num_attention_heads, module.config.num_key_value_heads
    q = module.q_proj(x).view(B, L, hq, D).transpose(1, 2)
    k = module.k_proj(x).view(B, L, hkv, D).transpose(1, 2)
    v = module.v_proj(x).view(B, L, hkv, D).transpose(1, 2)
    return q, k, v


def selftest_replay(device, dtype, tol, LEN=511, W=256, C=128, n_decode=300, seed=0, M=None):
    """ops/attn_vq.py:534-556 with an assertion: fast path vs the naive oracle, then ``n_decode`` generated
    tokens through the same module and cache, each checked against the oracle row of the whole sequence."""
    from vqtree_b200.attn_vq import AttentionMode, VectorQuantizedReRoPECache
    module = make_module(dtype, device, seed=seed)
    D = module.head_dim
    g = torch.Generator().manual_seed(seed + 1)
    codebook = torch.randn(2, C, D, generator=g) if M is None else torch.randn(2, M, C, D, generator=g)
    codebook = codebook.to(dtype).to(device)
    total = LEN + n_decode
    x = torch.randn(1, total, 128, generator=g).to(dtype).to(device)
    position_ids = torch.arange(total, device=device).unsqueeze(0)
    with torch.no_grad():
        q, k, v = project(module, x)
        want = oracle_rows(q, k, v, codebook.float(), W, dtype)
        cache = VectorQuantizedReRoPECache(W, codebook, False, attention_mode=AttentionMode.SORT_BASED_LINEAR)
        o_fast, weights, returned = module(hidden_states=x[:, :LEN], position_ids=position_ids[:, :LEN], past_key_value=cache)
        assert weights is None and returned is cache
        assert o_fast.shape == (1, LEN, 128)
        err = np.abs(_f(o_fast) - want[:, :LEN]).max()
        assert err <= tol, f"prefill max-abs {err}"
        # the prefill oracle of a longer sequence agrees with the shorter one on the common rows (causal), so the
        # generated tokens are checked against rows LEN.. of the same oracle run
        assert cache.get_seq_length(0) == LEN and cache.seen_tokens == LEN
        worst = 0.0
        for t in range(LEN, total):
            o, _, _ = module(hidden_states=x[:, t:t + 1], position_ids=position_ids[:, t:t + 1], past_key_value=cache)
            assert o.shape == (1, 1, 128)
            worst = max(worst, float(np.abs(_f(o)[:, 0] - want[:, t]).max()))
        assert worst <= tol, f"decode max-abs {worst}"
        assert cache.get_seq_length(0) == total and cache.seen_tokens == total
        # the other mode of the reference's self-test: an independent fp32 kernel on the same inputs
        cache2 = VectorQuantizedReRoPECache(W, codebook, False, attention_mode=AttentionMode.SLOW_REFERNECE)
        o_ref = module(hidden_states=x[:, :LEN], position_ids=position_ids[:, :LEN], past_key_value=cache2)[0]
        assert np.abs(_f(o_ref) - want[:, :LEN]).max() <= tol
        assert np.abs(_f(o_ref) - _f(o_fast)).max() <= 2 * tol
    return err, worst


def short_prefill_is_plain_causal(device, dtype, tol, W=128, L=200):
    """A prefill of W < L <= W + 128 tokens takes the reference's short-sequence path: plain causal attention
    over rotated q / k, no window (ops/attn_vq.py:231-248,445-476)."""
    from vqtree_b200.attn_vq import VectorQuantizedReRoPECache
    module = make_module(dtype, device, seed=3)
    D = module.head_dim
    g = torch.Generator().manual_seed(4)
    codebook = torch.randn(2, 128, D, generator=g).to(dtype).to(device)
    x = torch.randn(2, L, 128, generator=g).to(dtype).to(device)
    pos = torch.arange(L, device=device).unsqueeze(0).expand(2, L)
    with torch.no_grad():
        q, k, v = project(module, x)
        cos, sin = vo.rope_tables(L, D)
        rd = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dtype).float()
        q1, k1 = rd(vo.apply_rope(_f(q), cos, sin, np.arange(L))), rd(vo.apply_rope(_f(k), cos, sin, np.arange(L)))
        s = torch.einsum("bhid,bhjd->bhij", q1, k1) / D ** 0.5
        s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1), float("-inf"))
        want = torch.einsum("bhij,bhjd->bhid", torch.softmax(s, -1), v.float().cpu()).transpose(1, 2).reshape(2, L, -1)
        cache = VectorQuantizedReRoPECache(W, codebook)
        got = module(hidden_states=x, position_ids=pos, past_key_value=cache)[0]
        assert np.abs(_f(got) - want.numpy()).max() <= tol
        assert cache.get_seq_length(0) == L


def save_load_continues(device, dtype, tmp_path, LEN=520, W=128, n_decode=140):
    """Prefill, save the cache, reload it, and generate from both: identical outputs, token by token."""
    from vqtree_b200 import codebook_io
    from vqtree_b200.attn_vq import VectorQuantizedReRoPECache
    module = make_module(dtype, device, seed=5)
    g = torch.Generator().manual_seed(6)
    codebook = torch.randn(2, 2, 128, module.head_dim, generator=g).to(device)
    x = torch.randn(1, LEN + n_decode, 128, generator=g).to(dtype).to(device)
    with torch.no_grad():
        cache = VectorQuantizedReRoPECache(W, codebook)
        module(hidden_states=x[:, :LEN], past_key_value=cache)
        for t in range(LEN, LEN + 10):       # a few steps first, so that the window no longer starts at row 0
            module(hidden_states=x[:, t:t + 1], past_key_value=cache)
        codebook_io.save_cache(cache, tmp_path / "cache.pt")
        again = codebook_io.load_cache(tmp_path / "cache.pt", device=device)
        assert again.get_seq_length(0) == cache.get_seq_length(0) and again.seen_tokens == cache.seen_tokens
        for t in range(LEN + 10, LEN + n_decode):
            a = module(hidden_states=x[:, t:t + 1], past_key_value=cache)[0]
            b = module(hidden_states=x[:, t:t + 1], past_key_value=again)[0]
            assert torch.equal(a, b), f"token {t} differs after reload"


def tiny_llama_generate(device, dtype, tol, n_new=40, L=400, W=128):
    """A two-layer Llama built under ``use_rerope(o_proj=True)``: ``model.generate`` runs with the VQ cache, and the
    logits of an incremental run equal those of one prefill over the same tokens (cache bookkeeping, both
    layers)."""
    from transformers.models.llama import LlamaConfig, LlamaForCausalLM
    from vqtree_b200.attn_vq import LlamaFlashAttention2VectorQuantizedReRoPE, VectorQuantizedReRoPECache, use_rerope
    torch.manual_seed(7)
    config = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                         num_key_value_heads=1, vocab_size=97, max_position_embeddings=4096)
    with use_rerope(o_proj=True):
        model = LlamaForCausalLM(config).to(dtype).to(device).eval()
    assert all(isinstance(l.self_attn, LlamaFlashAttention2VectorQuantizedReRoPE) for l in model.model.layers)
    g = torch.Generator().manual_seed(8)
    codebook = torch.randn(1, 2, 128, 64, generator=g).to(device)
    ids = torch.randint(0, 97, (1, L), generator=g).to(device)
    with torch.no_grad():
        cache = VectorQuantizedReRoPECache(W, codebook)
        out = model.generate(ids, past_key_values=cache, max_new_tokens=n_new, do_sample=False, use_cache=True)
        assert out.shape == (1, L + n_new)
        assert cache.get_seq_length(0) == L + n_new - 1 and cache.get_seq_length(1) == L + n_new - 1
        # one prefill over the generated sequence reproduces the logits of the last incremental step
        cache_a = VectorQuantizedReRoPECache(W, codebook)
        step_logits = []
        lg = model(out[:, :L], past_key_values=cache_a, use_cache=True).logits[:, -1]
        step_logits.append(lg)
        for t in range(L, L + n_new - 1):
            step_logits.append(model(out[:, t:t + 1], past_key_values=cache_a, use_cache=True).logits[:, -1])
        full = model(out[:, :-1], past_key_values=VectorQuantizedReRoPECache(W, codebook), use_cache=True).logits
        for j, lg in enumerate(step_logits):
            ref = full[:, L - 1 + j]
            assert float((lg.float() - ref.float()).abs().max()) <= tol, f"step {j}"
        assert torch.equal(torch.stack(step_logits, 1).argmax(-1)[0], out[0, L:])
