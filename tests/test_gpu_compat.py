"""GPU tests of the mirrors of the reference's Python entry points, against golden vectors
produced by the reference itself (tests/golden/gen_golden.py)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_multi_head_single_quantize_matches_reference(golden_dir):
    from vqtree_b200.mini_vq import multi_head_single_quantize
    gd = np.load(golden_dir / "assign_a.npz")
    k, cb = torch.from_numpy(gd["k"]).cuda(), torch.from_numpy(gd["codebook"]).cuda()
    quantized, ids, onehot = multi_head_single_quantize(k, cb)
    assert ids.dtype == torch.int64 and ids.shape == k.shape[:3]
    assert onehot.shape == (*k.shape[:3], cb.shape[1]) and int(onehot.sum()) == ids.numel()
    assert (ids.cpu().numpy() != gd["ids"]).mean() < 1e-3
    np.testing.assert_array_equal(quantized[:, :, :8].cpu().numpy()[ids[:, :, :8].cpu().numpy() == gd["ids"][:, :, :8]],
                                  gd["quantized_head"][ids[:, :, :8].cpu().numpy() == gd["ids"][:, :, :8]])


def test_vq_attn_forward_on_reference_arguments(golden_dir):
    """Feed the exact tensors the reference handed to its fused kernel; compare with its merged output."""
    from vqtree_b200.fused_vq_attn import vq_attn_forward
    f = np.load(golden_dir / "fast_w128.npz")
    gd = np.load(golden_dir / "naive_w128.npz")
    cu = lambda a: torch.from_numpy(a).cuda()
    out = vq_attn_forward(cu(f["q1"]), cu(f["q2"]), cu(f["k1"]), cu(gd["codebook"]), cu(f["k_vq_cnt"]).float(), cu(gd["k"]),
                          cu(gd["v"]), cu(f["v_vq"]), cu(f["vi"]).long(), int(gd["window"]))
    np.testing.assert_allclose(out.cpu().numpy(), f["out"], atol=1e-4, rtol=0)
    np.testing.assert_allclose(out.cpu().numpy(), gd["out"], atol=1e-4, rtol=0)
    # bf16, the dtype the reference's kernels are written for (tolerance of its sibling self-tests)
    b = lambda a: torch.from_numpy(a).cuda().bfloat16()
    out16 = vq_attn_forward(b(f["q1"]), b(f["q2"]), b(f["k1"]), b(gd["codebook"]), cu(f["k_vq_cnt"]).bfloat16(), b(gd["k"]),
                            b(gd["v"]), b(f["v_vq"]), cu(f["vi"]).long(), int(gd["window"]))
    np.testing.assert_allclose(out16.float().cpu().numpy(), f["out"], atol=2e-2, rtol=0)


def test_local_flash_attn_func(golden_dir):
    from vqtree_b200.fused_local_attn_rerope import flash_attn_func
    f = np.load(golden_dir / "fast_w128.npz")
    gd = np.load(golden_dir / "naive_w128.npz")
    t = lambda a: torch.from_numpy(a).cuda().transpose(1, 2).contiguous()   # [B,L,H,D]
    o, lse = flash_attn_func(t(f["q1"]), t(f["q2"]), t(f["k1"]), t(gd["k"]), t(gd["v"]), int(gd["window"]), return_lse=True)
    assert o.shape == t(f["q1"]).shape
    np.testing.assert_allclose(o.transpose(1, 2).cpu().numpy(), f["o_local"], atol=1e-4, rtol=0)
    np.testing.assert_allclose(lse.cpu().numpy(), f["lse_local"], atol=1e-3, rtol=0)
    o16 = flash_attn_func(*(x.bfloat16() for x in (t(f["q1"]), t(f["q2"]), t(f["k1"]), t(gd["k"]), t(gd["v"]))), int(gd["window"]))
    np.testing.assert_allclose(o16.float().transpose(1, 2).cpu().numpy(), f["o_local"], atol=2e-2, rtol=0)


def test_long_prefilling_entry_point(golden_dir):
    from vqtree_b200.attn_vq import AttentionMode, VectorQuantizedReRoPECache, long_prefilling_sort_based_linear, BLOCK_SIZE
    assert BLOCK_SIZE == 128
    gd = np.load(golden_dir / "naive_w128.npz")
    q, k, v, cb = (torch.from_numpy(gd[n]).cuda() for n in ("q", "k", "v", "codebook"))
    B, H, L, D = q.shape
    cache = VectorQuantizedReRoPECache(int(gd["window"]), cb, False, attention_mode=AttentionMode.SORT_BASED_LINEAR)
    pos = torch.arange(L, device="cuda")[None].expand(B, -1)
    out = long_prefilling_sort_based_linear(q, k, v, pos, L, cache)
    assert out.shape == (B, L, H * D)
    want = torch.from_numpy(gd["out"]).transpose(1, 2).reshape(B, L, H * D)
    np.testing.assert_allclose(out.cpu().numpy(), want.numpy(), atol=1e-4, rtol=0)
    assert cache.get_seq_length(0) == L


@pytest.mark.parametrize("dtype,L0,T,hq,hkv,D", [(torch.bfloat16, 600, 330, 8, 2, 128), (torch.float32, 300, 140, 2, 2, 128),
                                                 (torch.bfloat16, 100, 40, 4, 4, 128), (torch.bfloat16, 400, 150, 4, 2, 64)])
def test_cache_prefill_then_decode_steps(dtype, L0, T, hq, hkv, D):
    """Prefill L0 tokens into the cache, then generate T more one at a time (the boundary moves at least
    twice in the long cases); every generated row must match the naive per-query attention over the whole sequence."""
    from oracle import vq_oracle as vo
    from vqtree_b200 import api
    from vqtree_b200.attn_vq import (AttentionMode, VectorQuantizedReRoPECache, dispatch_attn_impl, rope_cos_sin,
                                     rotate_half)
    B, M, K, W = 1, 2, 128, 256
    L = L0 + T
    g = torch.Generator(device="cpu").manual_seed(77)
    q = torch.randn(B, hq, L, D, generator=g).cuda().to(dtype)
    k = torch.randn(B, hkv, L, D, generator=g).cuda().to(dtype)
    v = torch.randn(B, hkv, L, D, generator=g).cuda().to(dtype)
    cb = (torch.randn(hkv, M, K, D, generator=g) * 0.7).to(dtype).float().cuda()
    cache = VectorQuantizedReRoPECache(W, cb, False, attention_mode=AttentionMode.SORT_BASED_LINEAR)
    pos = torch.arange(L, device="cuda")[None].expand(B, -1)
    got = [dispatch_attn_impl(q[:, :, :L0], k[:, :, :L0], v[:, :, :L0], pos[:, :L0], cache)]
    assert cache.get_seq_length(0) == L0
    with pytest.raises(AssertionError):   # a second prefill is refused like the reference does (ops/attn_vq.py:192-196)
        dispatch_attn_impl(q[:, :, :2], k[:, :, :2], v[:, :, :2], pos[:, :2], cache)
    for i in range(L0, L):
        got.append(dispatch_attn_impl(q[:, :, i:i + 1], k[:, :, i:i + 1], v[:, :, i:i + 1], pos[:, i:i + 1], cache))
    assert cache.get_seq_length(0) == L and cache.seen_tokens == L
    got = torch.cat(got, dim=1).float().cpu().numpy()

    cos, sin = rope_cos_sin(max(L, W + 2), D, q.device)
    rot = lambda x, c, s: (x.float() * c + rotate_half(x.float()) * s).to(dtype).float().cpu().numpy()
    q1, k1 = rot(q, cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)), rot(k, cos[pos].unsqueeze(1), sin[pos].unsqueeze(1))
    q2 = rot(q, cos[W + 1], sin[W + 1])
    codes = api.assign_codes(k.contiguous(), cb).cpu().numpy()
    want = vo.attn_naive(q1, q2, k1, k.float().cpu().numpy(), v.float().cpu().numpy(), cb.cpu().numpy(), codes, W)
    if L0 <= W + 128:
        # a short prefill takes the reference's short-sequence path: plain causal attention over rotated q / k
        # (ops/attn_vq.py:231-248,445-476); the generated rows follow the windowed definition again
        plain = vo.attn_naive(q1[:, :, :L0], q1[:, :, :L0], k1[:, :, :L0], k1[:, :, :L0], v.float().cpu().numpy()[:, :, :L0],
                              cb.cpu().numpy(), codes[:, :, :L0], W + 128)
        want[:, :, :L0] = plain
    want = want.transpose(0, 2, 1, 3).reshape(B, L, hq * D)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    np.testing.assert_allclose(got, want, atol=tol, rtol=0)
