"""The CPU oracle against golden vectors produced by the reference's own code.

The ``.npz`` files under tests/golden were written by tests/golden/gen_golden.py, which
executes the reference (ops/mini_vq.py, the naive loop and the host preparation in
ops/attn_vq.py, and the two Triton kernels under the interpreter).  These tests pin the M = 1
forms of the oracle to those outputs.
"""
import numpy as np
import pytest

from oracle import vq_oracle as vo

TIE_REL = 2.0 ** -18  # a code mismatch is tolerated only where the fp64 top-2 gap is below this * max|score|


def _load(golden_dir, name):
    return dict(np.load(golden_dir / name))


@pytest.mark.parametrize("name", ["assign_a.npz", "assign_b.npz"])
def test_assign_matches_reference_argmax(golden_dir, name):
    g = _load(golden_dir, name)
    k, cb, ids = g["k"], g["codebook"], g["ids"]
    codes = vo.assign_codes(k, cb[:, None])[..., 0]
    mism = codes != ids
    if mism.any():
        # both candidates must be within a near-tie of the fp64 maximum
        m_or, mx = vo.assign_margin(k, cb[:, None], codes[..., None])
        m_ref, _ = vo.assign_margin(k, cb[:, None], ids[..., None])
        tol = TIE_REL * mx[..., 0]
        assert (np.abs(m_or[..., 0])[mism] <= tol[mism]).all()
        assert (np.abs(m_ref[..., 0])[mism] <= tol[mism]).all()
    assert mism.mean() < 1e-3
    # the fp64 margin of every oracle code is non-negative up to rounding
    margin, mx = vo.assign_margin(k, cb[:, None], codes[..., None])
    assert (margin[..., 0] >= -TIE_REL * mx[..., 0]).all()
    # reconstruction rows the reference returned are the chosen codewords
    q = g["quantized_head"]
    B, H = q.shape[:2]
    for b in range(B):
        for h in range(H):
            np.testing.assert_array_equal(q[b, h], cb[h][ids[b, h, :8]])


def _rope_inputs(g):
    q, k, v, cb, W = g["q"], g["k"], g["v"], g["codebook"], int(g["window"])
    L, D = q.shape[2], q.shape[3]
    cos, sin = vo.rope_tables(max(L, W + 2), D)
    pos = np.arange(L)
    q1 = vo.apply_rope(q, cos, sin, pos)
    k1 = vo.apply_rope(k, cos, sin, pos)
    q2 = vo.apply_rope(q, cos, sin, np.full(L, W + 1))
    return q1, q2, k1, k, v, cb, W


@pytest.mark.parametrize("name", ["naive_selftest.npz", "naive_w128.npz"])
def test_naive_matches_reference_slow_impl(golden_dir, name):
    g = _load(golden_dir, name)
    q1, q2, k1, k3, v, cb, W = _rope_inputs(g)
    codes = vo.assign_codes(k3, cb[:, None])
    out = vo.attn_naive(q1, q2, k1, k3, v, cb[:, None], codes, W)
    np.testing.assert_allclose(out, g["out"], atol=2e-5, rtol=0)


def test_aggregates_and_fast_path_match_reference(golden_dir):
    g = _load(golden_dir, "naive_w128.npz")
    f = _load(golden_dir, "fast_w128.npz")
    q1, q2, k1, k3, v, cb, W = _rope_inputs(g)
    # the rotary helpers reproduce what the reference handed to its kernels
    np.testing.assert_allclose(q1, f["q1"], atol=2e-6)
    np.testing.assert_allclose(q2, f["q2"], atol=2e-6)
    np.testing.assert_allclose(k1, f["k1"], atol=2e-6)
    codes = vo.assign_codes(k3, cb[:, None])
    K = cb.shape[1]
    cnt, vsum = vo.build_aggregates(codes, v, K)
    # counts: the reference keeps the running count at the last row of every 128-block
    np.testing.assert_array_equal(cnt[:, :, :, 0, :], f["k_vq_cnt"])
    # value sums: row vi[n, c] of the reference's sorted prefix array is the sum over the members of c
    v_vq, vi = f["v_vq"], f["vi"]
    B, H, NB = vi.shape[:3]
    for b in range(B):
        for h in range(H):
            got = v_vq[b, h][vi[b, h]]  # [NB, K, D]
            mask = cnt[b, h, :, 0, :] > 0
            np.testing.assert_allclose(vsum[b, h, :, 0][mask], got[mask], atol=2e-4, rtol=0)
    out, lse = vo.attn_agg(q1, q2, k1, k3, v, cb[:, None], cnt, vsum, W, return_lse=True)
    np.testing.assert_allclose(out, f["out"], atol=2e-5, rtol=0)
    np.testing.assert_allclose(out, g["out"], atol=2e-5, rtol=0)
    # merged base-2 log-sum-exp of the two kernels
    l1, l2 = f["lse_local"], f["lse_far"]
    mx = np.maximum(l1, l2)
    merged = mx + np.log2(np.exp2(l1 - mx) + np.exp2(l2 - mx))
    np.testing.assert_allclose(lse, merged, atol=2e-4, rtol=0)


def test_agg_equals_naive_for_multiple_codebooks():
    rng = np.random.default_rng(5)
    B, Hq, Hkv, L, D, M, K, W = 1, 4, 2, 512, 32, 3, 128, 128
    q1 = rng.standard_normal((B, Hq, L, D), dtype=np.float32)
    q2 = rng.standard_normal((B, Hq, L, D), dtype=np.float32)
    k1 = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    k3 = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    cb = rng.standard_normal((Hkv, M, K, D), dtype=np.float32) * 0.4
    codes = vo.assign_codes(k3, cb)
    cnt, vsum = vo.build_aggregates(codes, v, K)
    a = vo.attn_naive(q1, q2, k1, k3, v, cb, codes, W)
    b = vo.attn_agg(q1, q2, k1, k3, v, cb, cnt, vsum, W)
    np.testing.assert_allclose(a, b, atol=3e-5, rtol=0)


def test_decode_equals_prefill_row():
    rng = np.random.default_rng(6)
    B, Hq, Hkv, L, D, M, K, W = 2, 4, 2, 640, 32, 2, 128, 128
    q1 = rng.standard_normal((B, Hq, L, D), dtype=np.float32)
    q2 = rng.standard_normal((B, Hq, L, D), dtype=np.float32)
    k1 = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    k3 = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    cb = rng.standard_normal((Hkv, M, K, D), dtype=np.float32) * 0.4
    codes = vo.assign_codes(k3, cb)
    cnt, vsum = vo.build_aggregates(codes, v, K)
    full = vo.attn_naive(q1, q2, k1, k3, v, cb, codes, W)
    for n in (100, 257, 500, 640):
        i = n - 1
        bd = max(0, (i - W) // 128 * 128)
        lb = max(0, i - W)
        use_far = bd > 0
        blk = bd // 128 - 1 if use_far else 0
        out = vo.decode(q1[:, :, i], q2[:, :, i], k1[:, :, bd:n], k3[:, :, bd:n], v[:, :, bd:n], cb,
                        cnt[:, :, blk], vsum[:, :, blk], n - bd, lb - bd, use_far=use_far)
        np.testing.assert_allclose(out, full[:, :, i], atol=3e-5, rtol=0)
