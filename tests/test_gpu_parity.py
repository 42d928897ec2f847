"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the golden vectors.

Tolerances (stated by the task): codes bit-exact; outputs max-abs <= 2e-2 in bf16 and <= 1e-4 in
fp32 against the naive oracle evaluated on the same (rounded) inputs.
"""
import numpy as np
import pytest
import torch

from oracle import vq_oracle as vo
from tests.vq_cases import make_case, oracle_prefill

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def api():
    assert torch.cuda.is_available(), "the gpu-marked tests need a CUDA device"
    from vqtree_b200 import api as _api
    return _api


def dev(t):
    return t.cuda() if t is not None else None


# ----------------------------------------------------------------------------- assignment

@pytest.mark.parametrize("B,Hkv,L,D,M,K,dtype,code_dtype", [
    (1, 8, 1024, 64, 2, 256, torch.float32, torch.uint8),      # config 1 shape
    (1, 8, 1024, 64, 1, 256, torch.float32, torch.int64),      # the reference's single-codebook case
    (2, 3, 640, 128, 4, 256, torch.bfloat16, torch.uint8),
    (1, 2, 333, 128, 4, 512, torch.bfloat16, torch.uint16),    # ragged length, 9-bit codes
    (1, 2, 64, 64, 3, 64, torch.float32, torch.int32),
])
def test_assign_codes_bit_exact(api, B, Hkv, L, D, M, K, dtype, code_dtype):
    g = torch.Generator().manual_seed(11 + L + K)
    k = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
    cb = torch.randn(Hkv, M, K, D, generator=g) * D ** -0.25
    want = vo.assign_codes(k.float().numpy(), cb.numpy())
    got = api.assign_codes(dev(k), dev(cb), out_dtype=code_dtype)
    assert got.dtype == code_dtype
    np.testing.assert_array_equal(got.cpu().to(torch.int64).numpy(), want)


def test_assign_codes_with_bias_and_strided_keys(api):
    g = torch.Generator().manual_seed(5)
    B, Hkv, L, D, M, K = 2, 2, 256, 64, 2, 128
    kfull = torch.randn(B, L, Hkv, D, generator=g)           # [B,L,H,D] storage, viewed as [B,H,L,D]
    k = kfull.transpose(1, 2)
    cb = torch.randn(Hkv, M, K, D, generator=g) * 0.4
    bias = -0.5 * (cb ** 2).sum(-1)                            # the L2 assignment rule
    want = vo.assign_codes(k.contiguous().numpy(), cb.numpy(), bias.numpy())
    got = api.assign_codes(dev(kfull).transpose(1, 2), dev(cb), dev(bias))
    np.testing.assert_array_equal(got.cpu().to(torch.int64).numpy(), want)


def test_assign_matches_reference_golden(api, golden_dir):
    for name in ("assign_a.npz", "assign_b.npz"):
        gd = np.load(golden_dir / name)
        k, cb, ids = torch.from_numpy(gd["k"]), torch.from_numpy(gd["codebook"]), gd["ids"]
        got = api.assign_codes(dev(k), dev(cb[:, None].contiguous())).cpu().to(torch.int64).numpy()[..., 0]
        mism = got != ids
        if mism.any():
            margin, mx = vo.assign_margin(gd["k"], gd["codebook"][:, None], ids[..., None])
            assert (np.abs(margin[..., 0])[mism] <= 2.0 ** -18 * mx[..., 0][mism]).all()
        assert mism.mean() < 1e-3


# ----------------------------------------------------------------------------- aggregates

@pytest.mark.parametrize("D,M,K,dtype", [(64, 2, 256, torch.float32), (128, 4, 256, torch.bfloat16),
                                         (128, 2, 512, torch.bfloat16), (64, 1, 128, torch.float32)])
def test_build_aggregates(api, D, M, K, dtype):
    B, Hkv, L = 2, 2, 768
    g = torch.Generator().manual_seed(3 + K)
    codes = torch.randint(0, K, (B, Hkv, L, M), generator=g)
    v = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
    cnt_w, vsum_w = vo.build_aggregates(codes.numpy(), v.float().numpy(), K, NB=5)
    cdt = torch.uint8 if K <= 256 else torch.uint16
    cnt, vsum = api.build_aggregates(dev(codes.to(cdt)), dev(v), K, nb=5)
    np.testing.assert_array_equal(cnt.cpu().numpy().reshape(cnt_w.shape), cnt_w.astype(np.float32))
    want = vsum_w.reshape(B, Hkv, 5, M * K, D)
    if dtype == torch.bfloat16:
        want = vo.round_bf16(want)
    np.testing.assert_array_equal(vsum.float().cpu().numpy(), want)  # same fp32 order -> bit-exact
    # fp32 master copy from bf16 values
    if dtype == torch.bfloat16:
        _, vs32 = api.build_aggregates(dev(codes.to(cdt)), dev(v), K, nb=5, out_dtype=torch.float32)
        np.testing.assert_array_equal(vs32.cpu().numpy(), vsum_w.reshape(B, Hkv, 5, M * K, D))


@pytest.mark.parametrize("D", [64, 128])
def test_build_aggregates_skewed_codes(api, D):
    """Every key of a block in one or two code rows (far more keys per row than the kernel stages at once)."""
    B, Hkv, L, M, K = 1, 2, 640, 3, 128
    g = torch.Generator().manual_seed(17)
    codes = torch.randint(0, K, (B, Hkv, L, M), generator=g)
    codes[:, 0, :, 0] = 5                                     # one row takes every key
    codes[:, 0, :, 1] = torch.where(torch.arange(L) % 3 == 0, 8, 15)  # two rows of one warp
    codes[:, 1, :128, 2] = 127
    v = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16)
    cnt_w, vsum_w = vo.build_aggregates(codes.numpy(), v.float().numpy(), K, NB=4)
    cnt, vsum = api.build_aggregates(dev(codes.to(torch.uint8)), dev(v), K, nb=4)
    np.testing.assert_array_equal(cnt.cpu().numpy().reshape(cnt_w.shape), cnt_w.astype(np.float32))
    np.testing.assert_array_equal(vsum.float().cpu().numpy(), vo.round_bf16(vsum_w.reshape(B, Hkv, 4, M * K, D)))


@pytest.mark.parametrize("D,M,K,cdt", [(128, 4, 256, torch.uint8), (64, 2, 512, torch.uint16), (128, 1, 1024, torch.int32),
                                       (128, 3, 8, torch.uint8)])
def test_build_aggregates_sorted_equals_scan(api, D, M, K, cdt):
    """The entry point with a workspace (every block's keys sorted by code first) and the one without it give the
    same counts and sums bit for bit - also on a strided view of the values and with skewed codes."""
    B, Hkv, L, nb = 2, 3, 1024, 7
    g = torch.Generator().manual_seed(5 + K)
    codes = torch.randint(0, K, (B, Hkv, L, M), generator=g)
    codes[0, 1, 128:512, 0] = K - 1                            # a row with far more keys than are staged at once
    codes[1, 2, :, M - 1] = torch.arange(L) % 5               # five rows of one warp share every block
    store = torch.randn(B, L, Hkv, D + 8, generator=g).to(torch.bfloat16)
    v = dev(store)[..., :D].permute(0, 2, 1, 3)               # [B,Hkv,L,D] view of [B,L,Hkv,D+8] storage
    c = dev(codes.to(cdt))
    cnt_a, vsum_a = api.build_aggregates(c, v, K, nb=nb, impl="scan")
    cnt_b, vsum_b = api.build_aggregates(c, v, K, nb=nb)
    torch.cuda.synchronize()
    api.check_status()
    assert torch.equal(cnt_a, cnt_b)
    assert torch.equal(vsum_a.view(torch.int16), vsum_b.view(torch.int16))
    cnt_w, vsum_w = vo.build_aggregates(codes.numpy(), v.float().cpu().numpy(), K, NB=nb)
    np.testing.assert_array_equal(cnt_b.cpu().numpy().reshape(cnt_w.shape), cnt_w.astype(np.float32))
    np.testing.assert_array_equal(vsum_b.float().cpu().numpy(), vo.round_bf16(vsum_w.reshape(B, Hkv, nb, M * K, D)))


@pytest.mark.parametrize("vdt,D,M,K,extra", [(torch.bfloat16, 128, 4, 256, 1), (torch.bfloat16, 64, 2, 512, 0),
                                             (torch.bfloat16, 128, 1, 1024, 1), (torch.float32, 64, 2, 128, 1),
                                             (torch.float16, 128, 2, 256, 1)])
def test_build_aggregates_state_equals_cache_advance(api, vdt, D, M, K, extra):
    """The decode-phase state taken from the aggregate pass (fp32 counts and sums of the first state_blocks * 128 keys)
    equals the cache-advance kernel applied to those keys from zero, bit for bit, and the snapshots are unchanged -
    on the sorted path (bf16) and on the inputs it does not cover (f32 / f16 values)."""
    B, Hkv, L, nb = 2, 3, 1024 + 64, 7
    sb = nb + extra
    g = torch.Generator().manual_seed(11 + K)
    codes = torch.randint(0, K, (B, Hkv, L, M), generator=g)
    codes[0, 1, 128:512, 0] = K - 1
    store = torch.randn(B, L, Hkv, D + 8, generator=g).to(vdt)
    v = dev(store)[..., :D].permute(0, 2, 1, 3)
    c = dev(codes.to(torch.int32))
    cnt_a, vsum_a = api.build_aggregates(c, v, K, nb=nb)
    cnt_b, vsum_b, s_cnt, s_vsum = api.build_aggregates(c, v, K, nb=nb, state_blocks=sb)
    want_cnt = torch.zeros(B, Hkv, M * K, device="cuda")
    want_vsum = torch.zeros(B, Hkv, M * K, D, device="cuda")
    api.cache_advance(c[:, :, :sb * 128], v[:, :, :sb * 128], K, want_cnt, want_vsum, None)
    torch.cuda.synchronize()
    api.check_status()
    assert torch.equal(cnt_a, cnt_b) and torch.equal(vsum_a.float(), vsum_b.float())
    assert torch.equal(s_cnt, want_cnt)
    assert torch.equal(s_vsum.view(torch.int32), want_vsum.view(torch.int32))
    assert float(s_cnt.sum()) == B * Hkv * M * sb * 128


def test_build_aggregates_state_rejects_bad_block_counts(api):
    B, Hkv, L, M, K, D = 1, 2, 512, 2, 64, 128
    codes = dev(torch.randint(0, K, (B, Hkv, L, M)).to(torch.uint8))
    v = dev(torch.randn(B, Hkv, L, D).to(torch.bfloat16))
    with pytest.raises(AssertionError):
        api.build_aggregates(codes, v, K, nb=3, state_blocks=2)      # fewer blocks than snapshots
    with pytest.raises(AssertionError):
        api.build_aggregates(codes, v, K, nb=3, state_blocks=5)      # beyond the sequence
    from vqtree_b200 import native
    cnt = torch.empty(B, Hkv, 3, M * K, device="cuda")
    vsum = torch.empty(B, Hkv, 3, M * K, D, device="cuda", dtype=torch.bfloat16)
    s_cnt = torch.empty(B, Hkv, M * K, device="cuda")
    s_vsum = torch.empty(B, Hkv, M * K, D, device="cuda")
    d = native.desc
    args = (d(codes), d(v), K, d(cnt), d(vsum), d(s_cnt), d(s_vsum))
    assert native.lib.vqattn_build_aggregates_state(*args, 2, None, 0, None, None) == -1   # VQ_EINVAL_SHAPE
    assert native.lib.vqattn_build_aggregates_state(*args, 5, None, 0, None, None) == -1   # VQ_EINVAL_SHAPE
    assert native.lib.vqattn_build_aggregates_state(d(codes), d(v), K, d(cnt), d(vsum), None, d(s_vsum), 3, None, 0, None, None) \
        == -7   # VQ_EINVAL_ARG


def test_build_aggregates_sorted_reports_codes_out_of_range(api):
    """A code outside [0, K) is left out of every row and raises the status word; the other keys are summed as usual."""
    B, Hkv, L, M, K, D, nb = 1, 2, 512, 2, 64, 128, 4
    g = torch.Generator().manual_seed(23)
    codes = torch.randint(0, K, (B, Hkv, L, M), generator=g)
    v = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16)
    bad = codes.clone()
    bad[0, 1, 200, 1] = 200                                    # >= K
    keep = torch.ones(B, Hkv, L, M, dtype=torch.bool)
    keep[0, 1, 200, 1] = False
    cnt, vsum = api.build_aggregates(dev(bad.to(torch.uint8)), dev(v), K, nb=nb)
    torch.cuda.synchronize()
    with pytest.raises(Exception):
        api.check_status()
    # expected: the same sums with that (key, codebook) pair removed
    onehot = torch.nn.functional.one_hot(codes, K).float() * keep[..., None]          # [B,Hkv,L,M,K]
    want_cnt = onehot.reshape(B, Hkv, nb, 128, M * K).sum(3).cumsum(2)
    np.testing.assert_array_equal(cnt.cpu().numpy(), want_cnt.numpy())
    api.check_status()                                         # the word was reset by the failed check


def test_gather_aggregates_from_reference_format(api, golden_dir):
    f = np.load(golden_dir / "fast_w128.npz")
    v_vq, vi = torch.from_numpy(f["v_vq"]), torch.from_numpy(f["vi"]).to(torch.int64)
    nb = vi.shape[2]
    got = api.gather_aggregates(dev(v_vq), dev(vi), nb).cpu().numpy()
    B, H = vi.shape[:2]
    for b in range(B):
        for h in range(H):
            np.testing.assert_array_equal(got[b, h], f["v_vq"][b, h][f["vi"][b, h]])
    # with the counts: rows of codes without members come out as zeros
    cnt = torch.from_numpy(f["k_vq_cnt"]).float()
    assert (cnt == 0).any()
    got0 = api.gather_aggregates(dev(v_vq), dev(vi), nb, dev(cnt)).cpu().numpy()
    keep = (f["k_vq_cnt"] > 0)[..., None]
    np.testing.assert_array_equal(got0, np.where(keep, got, 0.0))


# ----------------------------------------------------------------------------- prefill

def _run_prefill(api, case, impl):
    d = {k: dev(t) if isinstance(t, torch.Tensor) else t for k, t in case.items()}
    q2 = d["q1"] if case["q2"] is case["q1"] else d["q2"]
    k3 = d["k1"] if case["k3"] is case["k1"] else d["k3"]
    out, st = api.vq_attention_prefill(d["q1"], q2, d["k1"], k3, d["v"], d["cb"], case["W"], impl=impl, return_state=True)
    torch.cuda.synchronize()
    api.check_status()
    return out.float().cpu().numpy(), st


PREFILL_CASES = [
    # B, Hq, Hkv, L,   D,  M, K,   W,  seed, rerope, dtype
    (1, 8, 8, 1024, 64, 2, 256, 128, 0, False, torch.float32),    # config 1
    (1, 8, 8, 1024, 64, 1, 256, 128, 0, True, torch.float32),     # config 1 shape, reference-pinned M = 1, ReRoPE
    (1, 4, 2, 896, 128, 2, 128, 256, 7, True, torch.float32),     # GQA, D = 128
    (1, 2, 2, 700, 64, 1, 128, 128, 8, True, torch.float32),      # ragged tail (L % 128 != 0)
    (1, 2, 2, 200, 64, 1, 128, 128, 9, True, torch.float32),      # shorter than window + 128: no far part
    (1, 4, 4, 1024, 128, 4, 256, 256, 1, False, torch.bfloat16),  # config 2 shape, scaled down
    (2, 4, 2, 1024, 128, 4, 512, 128, 3, True, torch.bfloat16),   # config 4 shape, scaled down, GQA
    (1, 2, 2, 717, 64, 2, 128, 128, 4, True, torch.bfloat16),     # ragged, D = 64
    (1, 2, 2, 128, 128, 1, 128, 128, 11, True, torch.bfloat16),   # a single query tile
    (1, 2, 1, 300, 128, 2, 128, 128, 12, True, torch.bfloat16),   # three tiles (odd: the last pair has one), ragged, GQA
    (1, 2, 2, 1664, 128, 2, 128, 256, 13, False, torch.bfloat16), # thirteen tiles, far part from tile 3 on
]


@pytest.mark.parametrize("B,Hq,Hkv,L,D,M,K,W,seed,rerope,dtype", PREFILL_CASES)
@pytest.mark.parametrize("impl", ["simt", "tensor"])
def test_prefill_matches_naive_oracle(api, impl, B, Hq, Hkv, L, D, M, K, W, seed, rerope, dtype):
    if impl.startswith("tensor") and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel computes in bf16")
    case = make_case(B, Hq, Hkv, L, D, M, K, W, seed, rerope, dtype)
    want, codes = oracle_prefill(case)
    got, st = _run_prefill(api, case, impl)
    if st["codes"] is not None:
        np.testing.assert_array_equal(st["codes"].cpu().to(torch.int64).numpy(), codes)
    err = np.abs(got - want).max()
    assert np.isfinite(got).all()
    assert err <= TOL[dtype], f"max-abs error {err}"


def test_prefill_matches_reference_golden_output(api, golden_dir):
    """The reference's own naive loop and fast path (fp32, M = 1) on its inputs."""
    gd = np.load(golden_dir / "naive_w128.npz")
    W = int(gd["window"])
    q, k, v, cb = (torch.from_numpy(gd[n]) for n in ("q", "k", "v", "codebook"))
    L, D = q.shape[2], q.shape[3]
    cos, sin = vo.rope_tables(max(L, W + 2), D)
    pos = np.arange(L)
    q1 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, pos))
    k1 = torch.from_numpy(vo.apply_rope(k.numpy(), cos, sin, pos))
    q2 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, np.full(L, W + 1)))
    out = api.vq_attention_prefill(dev(q1), dev(q2), dev(k1), dev(k), dev(v), dev(cb[:, None].contiguous()), W)
    np.testing.assert_allclose(out.cpu().numpy(), gd["out"], atol=1e-4, rtol=0)
    fast = np.load(golden_dir / "fast_w128.npz")
    np.testing.assert_allclose(out.cpu().numpy(), fast["out"], atol=1e-4, rtol=0)


def test_prefill_lse_and_local_only(api, golden_dir):
    f = np.load(golden_dir / "fast_w128.npz")
    gd = np.load(golden_dir / "naive_w128.npz")
    W = int(gd["window"])
    q1, q2, k1 = (dev(torch.from_numpy(f[n])) for n in ("q1", "q2", "k1"))
    k3, v = dev(torch.from_numpy(gd["k"])), dev(torch.from_numpy(gd["v"]))
    out, lse = api.prefill_from_aggregates(q1, q2, k1, k3, v, None, None, None, W, return_lse=True)
    np.testing.assert_allclose(out.cpu().numpy(), f["o_local"], atol=1e-4, rtol=0)
    np.testing.assert_allclose(lse.cpu().numpy(), f["lse_local"], atol=1e-3, rtol=0)


# ----------------------------------------------------------------------------- decode

@pytest.mark.parametrize("B,Hq,Hkv,D,M,K,W,dtype,cb_f32", [
    (2, 4, 4, 128, 2, 128, 256, torch.bfloat16, True),
    (2, 8, 2, 128, 2, 128, 128, torch.bfloat16, False),   # GQA group of 4
    (1, 6, 2, 64, 1, 128, 128, torch.float32, True),      # group of 3 -> one head per CTA
    (3, 2, 1, 64, 2, 256, 128, torch.bfloat16, True),
    (2, 4, 4, 128, 2, 128, 256, torch.bfloat16, False),   # tensor-core decode kernel, one query head per kv head
    (1, 16, 2, 128, 1, 256, 256, torch.bfloat16, False),  # tensor-core decode kernel, group of 8
    (1, 3, 1, 128, 3, 128, 128, torch.bfloat16, False),   # tensor-core decode kernel, group of 3
])
def test_decode_matches_oracle_and_prefill_row(api, B, Hq, Hkv, D, M, K, W, dtype, cb_f32):
    L = 1024
    case = make_case(B, Hq, Hkv, L, D, M, K, W, 21, True, dtype)
    f = lambda t: t.float().numpy()
    cb = case["cb"].numpy()
    codes = vo.assign_codes(f(case["k3"]), cb)
    cnt, vsum = vo.build_aggregates(codes, f(case["v"]), K)
    cb_o = cb if (cb_f32 or dtype == torch.float32) else vo.round_bf16(cb)
    full = vo.attn_naive(f(case["q1"]), f(case["q2"]), f(case["k1"]), f(case["k3"]), f(case["v"]), cb_o, codes, W)
    ws = api.decode_workspace(B, Hq, Hkv, D, "cuda")
    for n in (W // 2, W + 130, 777, L):
        i = n - 1
        bd = max(0, (i - W) // 128 * 128)
        lb = max(0, i - W)
        far = bd > 0
        blk = bd // 128 - 1 if far else 0
        cnt_n = torch.from_numpy(cnt[:, :, blk].reshape(B, Hkv, M * K).astype(np.float32))
        vs_n = torch.from_numpy(vsum[:, :, blk].reshape(B, Hkv, M * K, D))
        vs_n = vs_n.to(dtype)
        cbk = torch.from_numpy(cb.reshape(Hkv, M * K, D))
        cbk = cbk if (cb_f32 or dtype == torch.float32) else cbk.to(dtype)
        # window buffers with slack rows beyond n_valid
        Nwin = W + 128 + 8
        def win(t):
            w = torch.zeros(B, Hkv, Nwin, D, dtype=dtype)
            w[:, :, : n - bd] = t[:, :, bd:n]
            return dev(w)
        got = api.vq_attention_decode(dev(case["q1"][:, :, i].contiguous()), dev(case["q2"][:, :, i].contiguous()),
                                      win(case["k1"]), win(case["k3"]), win(case["v"]),
                                      dev(cbk) if far else None, dev(cnt_n) if far else None, dev(vs_n) if far else None,
                                      n_valid=n - bd, n_bd=lb - bd, workspace=ws)
        want = vo.decode(f(case["q1"][:, :, i]), f(case["q2"][:, :, i]), f(case["k1"][:, :, bd:n]), f(case["k3"][:, :, bd:n]),
                         f(case["v"][:, :, bd:n]), cb_o, cnt[:, :, blk], f(vs_n).reshape(B, Hkv, M, K, D),
                         n - bd, lb - bd, use_far=far)
        tol = TOL[dtype]
        np.testing.assert_allclose(got.float().cpu().numpy(), want, atol=tol, rtol=0)
        np.testing.assert_allclose(got.float().cpu().numpy(), full[:, :, i], atol=tol, rtol=0)


def test_cache_advance(api):
    B, Hkv, D, M, K, n_new = 2, 2, 128, 2, 128, 128
    g = torch.Generator().manual_seed(31)
    codes0 = torch.randint(0, K, (B, Hkv, 256, M), generator=g)
    v0 = torch.randn(B, Hkv, 256, D, generator=g).bfloat16()
    cnt_w, vsum_w = vo.build_aggregates(codes0.numpy(), v0.float().numpy(), K, NB=2)
    cnt = dev(torch.from_numpy(cnt_w[:, :, 0].reshape(B, Hkv, M * K).astype(np.float32)))
    vs32 = dev(torch.from_numpy(vsum_w[:, :, 0].reshape(B, Hkv, M * K, D)))
    shadow = vs32.bfloat16()
    api.cache_advance(dev(codes0[:, :, 128:].to(torch.uint8).contiguous()), dev(v0[:, :, 128:].contiguous()), K, cnt, vs32, shadow)
    np.testing.assert_array_equal(cnt.cpu().numpy(), cnt_w[:, :, 1].reshape(B, Hkv, M * K).astype(np.float32))
    np.testing.assert_array_equal(vs32.cpu().numpy(), vsum_w[:, :, 1].reshape(B, Hkv, M * K, D))
    np.testing.assert_array_equal(shadow.float().cpu().numpy(), vo.round_bf16(vsum_w[:, :, 1].reshape(B, Hkv, M * K, D)))


# ----------------------------------------------------------------------------- error behaviour on the device

def test_errors_are_reported_not_crashed(api):
    from vqtree_b200.native import VqError
    k = torch.zeros(1, 2, 128, 64, device="cuda")
    with pytest.raises(VqError) as e:
        api.assign_codes(k, torch.zeros(2, 1, 100, 64, device="cuda"))      # K % 64 != 0
    assert e.value.status == -8
    with pytest.raises(VqError) as e:
        api.assign_codes(k, torch.zeros(3, 1, 128, 64, device="cuda"))      # head count mismatch
    assert e.value.status == -1
    with pytest.raises(VqError) as e:
        api.assign_codes(k, torch.zeros(2, 1, 512, 64, device="cuda"), out_dtype=torch.uint8)  # 9-bit codes into uint8
    assert e.value.status == -2
    q = torch.zeros(1, 2, 256, 64, device="cuda")
    with pytest.raises(VqError) as e:
        api.prefill_from_aggregates(q, q, q, q, q, None, None, None, window=100)  # window % 128 != 0
    assert e.value.status == -7


# ----------------------------------------------------------------------------- tensor-core assignment

@pytest.mark.parametrize("B,Hkv,L,D,M,K", [
    (1, 4, 2048, 128, 4, 256),     # config 2 shape, scaled down
    (2, 2, 700, 128, 4, 512),      # config 4 codebooks (9-bit codes), ragged length
    (1, 2, 1024, 128, 8, 256),     # config 5 codebooks
    (1, 3, 515, 64, 2, 128),       # D = 64
    (1, 1, 128, 128, 1, 64),       # single chunk
    (1, 2, 900, 128, 3, 384),      # three 128-codeword chunks, one key tile per CTA
    (2, 1, 640, 64, 2, 512),       # D = 64 with 9-bit codes
    (1, 2, 385, 128, 2, 128),      # odd number of key tiles: the last CTA has one
    (1, 2, 1500, 128, 1, 1024),    # one codebook of 1024 (the reference's format): four chunks through a score region of two
    (2, 1, 600, 128, 3, 1024),     # ... with residual codebooks
    (1, 2, 513, 64, 2, 1024),      # ... D = 64
])
def test_assign_tensor_path_is_bit_exact(api, B, Hkv, L, D, M, K):
    g = torch.Generator().manual_seed(77 + L + K + M)
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16()
    cb = torch.randn(Hkv, M, K, D, generator=g) * D ** -0.25
    want = vo.assign_codes(k.float().numpy(), cb.numpy())
    got = api.assign_codes(dev(k), dev(cb), out_dtype=torch.int32, impl="auto")
    torch.cuda.synchronize()
    api.check_status()
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    simt = api.assign_codes(dev(k), dev(cb), out_dtype=torch.int32, impl="simt")
    np.testing.assert_array_equal(simt.cpu().numpy(), want)


def test_assign_tensor_path_ties_zero_keys_and_bias(api):
    """Exact ties (duplicated codewords), all-zero keys, near-duplicates and a bias: the first maximum wins."""
    g = torch.Generator().manual_seed(5150)
    B, Hkv, L, D, M, K = 1, 2, 512, 128, 3, 128
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16()
    k[:, :, 10:20] = 0                                   # every score ties at zero
    cb = torch.randn(Hkv, M, K, D, generator=g) * 0.3
    cb[:, :, 64:96] = cb[:, :, 0:32]                      # exact duplicates: ties between c and c + 64
    cb[:, :, 100] = cb[:, :, 7] * (1 + 2 ** -22)          # a near-duplicate, far inside the error bound
    bias = torch.randn(Hkv, M, K, generator=g) * 0.1
    bias[:, :, 64:96] = bias[:, :, 0:32]
    for bs in (None, bias):
        want = vo.assign_codes(k.float().numpy(), cb.numpy(), None if bs is None else bs.numpy())
        got = api.assign_codes(dev(k), dev(cb), dev(bs), out_dtype=torch.int32)
        torch.cuda.synchronize()
        api.check_status()
        np.testing.assert_array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("kind", ["heavy_tail", "low_rank", "near_duplicates", "tiny_codebook", "huge_norms", "all_equal_keys",
                                  "near_duplicates_k1024", "heavy_tail_k1024", "near_duplicates_k512", "low_rank_k512",
                                  "all_equal_keys_k512", "close_pairs_k512", "close_pairs_k1024"])
def test_assign_tensor_path_adversarial_distributions(api, kind):
    """Data that stresses the error bound and the candidate records of the tensor-core assignment: heavy-tailed
    keys, keys in a low-dimensional subspace, codebooks full of near-duplicates (many candidates per key), codewords
    far smaller / far larger than the keys, identical keys.  Codes must equal the exact kernel's on every key (device
    comparison) and the oracle's on a slice."""
    g = torch.Generator().manual_seed(900 + len(kind) * 7 + ord(kind[0]))
    B, Hkv, L, D, M, K = 2, 3, 3000, 128, 4, 256
    if kind.endswith("_k1024"):
        kind, M, K = kind[:-6], 2, 1024
    elif kind.endswith("_k512"):       # four codebooks of 512: two chunks in rounds, with the residual chain
        kind, M, K = kind[:-5], 4, 512
    k = torch.randn(B, Hkv, L, D, generator=g)
    cb = torch.randn(Hkv, M, K, D, generator=g) * D ** -0.25
    if kind == "heavy_tail":
        k = k * torch.exp(2.0 * torch.randn(B, Hkv, L, 1, generator=g))
    elif kind == "low_rank":
        basis = torch.randn(4, D, generator=g)
        k = torch.randn(B, Hkv, L, 4, generator=g) @ basis
        cb = (torch.randn(Hkv, M, K, 4, generator=g) @ basis) * 0.3
    elif kind == "near_duplicates":
        base = torch.randn(Hkv, M, 16, D, generator=g) * D ** -0.25
        cb = base.repeat_interleave(K // 16, dim=2) * (1 + 2 ** -20 * torch.randn(Hkv, M, K, 1, generator=g))
        cb[:, :, 1::2] = cb[:, :, 0::2]                      # exact duplicates too: first index must win
    elif kind == "close_pairs":
        # every codeword has one near-twin 2^-16 away, in another chunk of 256 codes: the two candidates of a doubtful
        # key then come from different rounds through the score region
        half = cb[:, :, :K // 2]
        cb = torch.cat([half, half * (1 + 2 ** -16 * torch.randn(Hkv, M, K // 2, 1, generator=g))], dim=2)
    elif kind == "tiny_codebook":
        cb = cb * 1e-3
    elif kind == "huge_norms":
        cb = cb * 50.0
        k = k * 20.0
    elif kind == "all_equal_keys":
        k = k[:, :, :1].expand(B, Hkv, L, D).contiguous()
    k = k.bfloat16()
    got = api.assign_codes(dev(k), dev(cb), out_dtype=torch.int32, impl="auto")
    exact = api.assign_codes(dev(k), dev(cb), out_dtype=torch.int32, impl="simt")
    torch.cuda.synchronize()
    api.check_status()
    assert torch.equal(got, exact), f"{int((got != exact).sum())} codes differ"
    want = vo.assign_codes(k[:, :, :300].float().numpy(), cb.numpy())
    np.testing.assert_array_equal(got[:, :, :300].cpu().numpy(), want)


# ------------------------------------------------------------------ host-buffer entry (pipelined copies)
@pytest.mark.gpu
@pytest.mark.parametrize("B,Hq,Hkv,rerope,chunks", [(2, 8, 4, True, 8), (1, 6, 6, False, 4), (1, 4, 2, False, 1)])
def test_prefill_host_pipeline_equals_device_path(api, B, Hq, Hkv, rerope, chunks):
    """Chunked, stream-pipelined host entry == one device call on the same inputs, bit for bit."""
    case = make_case(B, Hq, Hkv, 1024, 128, 2, 128, 256, 31, rerope, torch.bfloat16)
    names = ("q1", "q2", "k1", "k3", "v")
    d = {n: dev(case[n]) for n in names}
    if not rerope:
        d["q2"], d["k3"] = d["q1"], d["k1"]
    cb = dev(case["cb"])
    want = api.vq_attention_prefill(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], cb, case["W"])
    h = {n: case[n].pin_memory() for n in names}
    if not rerope:
        h["q2"], h["k3"] = h["q1"], h["k1"]
    got = api.vq_attention_prefill_host(h["q1"], h["q2"], h["k1"], h["k3"], h["v"], cb, case["W"], chunks=chunks)
    api.check_status()
    assert not got.is_cuda and got.is_pinned()
    assert torch.equal(got, want.cpu())
    # unpinned inputs and a second call into the same output buffer
    got2 = api.vq_attention_prefill_host(case["q1"], case["q2"] if rerope else case["q1"], case["k1"],
                                         case["k3"] if rerope else case["k1"], case["v"], cb, case["W"], out=got)
    assert got2 is got and torch.equal(got2, want.cpu())


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64), (torch.bfloat16, 64)])
def test_rope_matches_elementwise_expression_and_oracle(dtype, D):
    """RoPE kernel against the element-wise expression the reference uses (ops/attn_vq.py:55-64,296-299,402-407):
    bit-exact against the same fp32 arithmetic in PyTorch, and within rounding of the oracle's float64 tables."""
    from oracle import vq_oracle as vo
    from vqtree_b200 import api
    from vqtree_b200.attn_vq import rope_cos_sin, rotate_half
    B, H, L, W = 2, 3, 333, 128
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(B, H, L, D, generator=g).cuda().to(dtype)
    pos = torch.stack([torch.arange(L), torch.arange(L).flip(0)]).cuda()
    cos, sin = rope_cos_sin(L, D, x.device)
    ref = lambda c, s: (x.float() * c + rotate_half(x.float()) * s).to(dtype)
    got_pos, got_const = api.rope(x, pos, const_pos=W + 1)
    assert torch.equal(got_pos, ref(cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)))
    assert torch.equal(got_const, ref(cos[W + 1], sin[W + 1]))
    plain, none = api.rope(x)                       # positions 0..L-1, no constant-position output
    assert none is None and torch.equal(plain[0], got_pos[0])
    only_const = api.rope(x[:, :, 5:9], const_pos=7, want_pos=False)   # a strided view, constant position only
    assert only_const[0] is None and torch.equal(only_const[1], ref(cos[7], sin[7])[:, :, 5:9])
    oc, osn = vo.rope_tables(L, D)
    want = vo.apply_rope(x.float().cpu().numpy(), oc, osn, pos.cpu().numpy()[:, None, :])
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    np.testing.assert_allclose(got_pos.float().cpu().numpy(), want, atol=tol, rtol=0)
    api.check_status()


def test_rope_reports_positions_outside_the_tables():
    from vqtree_b200 import api, native
    x = torch.randn(1, 1, 16, 64, device="cuda")
    pos = torch.arange(16, device="cuda")[None] + 10**6   # far beyond any table built so far (tables are cached and only grow)
    api.rope(x, pos, n_pos=32)
    with pytest.raises(native.VqError) as e:
        api.check_status()
    assert e.value.status == -7      # an invalid argument, not a time-out
    api.check_status()   # the word was cleared


def test_rope_qk_and_decode_append_match_the_rope_kernel():
    """The fused launches (q and k of a prefill; the per-token rotate-and-append of a decode) produce bit for bit
    what the single-tensor kernel produces, on [B,L,H,D] storage viewed as [B,H,L,D]."""
    from vqtree_b200 import api
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        B, L, Hq, Hkv, D, W = 2, 77, 4, 2, 128, 128
        g = torch.Generator(device="cpu").manual_seed(3)
        q = torch.randn(B, L, Hq, D, generator=g).cuda().to(dtype).transpose(1, 2)
        k = torch.randn(B, L, Hkv, D, generator=g).cuda().to(dtype).transpose(1, 2)
        v = torch.randn(B, L, Hkv, D, generator=g).cuda().to(dtype).transpose(1, 2)
        pos = (torch.arange(L) + 5)[None].expand(B, L).cuda()
        q1, q2, k1 = api.rope_qk(q, k, pos, const_pos=W + 1, like_input=True)
        assert q1.stride() == q.stride() and k1.stride() == k.stride()
        wq1, wq2 = api.rope(q.contiguous(), pos, const_pos=W + 1)
        wk1, _ = api.rope(k.contiguous(), pos)
        assert torch.equal(q1, wq1) and torch.equal(q2, wq2) and torch.equal(k1, wk1)
        # one token into row 9 of window caches
        wins = [torch.zeros(B, Hkv, 32, D, dtype=dtype, device="cuda") for _ in range(3)]
        oq1, oq2 = torch.empty(B, Hq, 1, D, dtype=dtype, device="cuda"), torch.empty(B, Hq, 1, D, dtype=dtype, device="cuda")
        t = 40
        api.decode_append(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], t + 5, W + 1, oq1, oq2, *wins, row=9)
        assert torch.equal(oq1[:, :, 0], wq1[:, :, t]) and torch.equal(oq2[:, :, 0], wq2[:, :, t])
        assert torch.equal(wins[0][:, :, 9], wk1[:, :, t]) and torch.equal(wins[1][:, :, 9], k[:, :, t]) and torch.equal(wins[2][:, :, 9], v[:, :, t])
        assert float(wins[0][:, :, :9].abs().max()) == 0 and float(wins[2][:, :, 10:].abs().max()) == 0
        # positions from a device tensor instead of the scalar
        api.decode_append(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], 0, W + 1, oq1, oq2, *wins, row=10,
                          positions=pos[:, t].contiguous(), n_pos=L + 6)
        assert torch.equal(wins[0][:, :, 10], wk1[:, :, t])
    api.check_status()


# ----------------------------------------------------------------------------- fp16 (the reference's self-test dtype)

@pytest.mark.parametrize("impl", ["simt", "tensor"])
@pytest.mark.parametrize("B,Hq,Hkv,L,D,M,K,W,seed,rerope", [
    (1, 2, 2, 511, 64, 1, 128, 256, 0, True),      # the reference's self-test shape (ops/attn_vq.py:534-556)
    (1, 4, 2, 1024, 128, 2, 256, 256, 5, True),    # GQA, D = 128, two codebooks
    (2, 2, 2, 700, 128, 4, 128, 128, 6, False),    # ragged, plain RoPE
])
def test_prefill_fp16_matches_naive_oracle(api, impl, B, Hq, Hkv, L, D, M, K, W, seed, rerope):
    case = make_case(B, Hq, Hkv, L, D, M, K, W, seed, rerope, torch.float16)
    want, codes = oracle_prefill(case)
    got, st = _run_prefill(api, case, impl)
    np.testing.assert_array_equal(st["codes"].cpu().to(torch.int64).numpy(), codes)
    assert st["vsum"] is None or st["vsum"].dtype == torch.float16
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-2


@pytest.mark.parametrize("B,Hq,Hkv,W,MK", [(3, 24, 8, 900, 512), (8, 32, 8, 2112, 2048)])
def test_decode_partial_merge_is_deterministic(api, B, Hq, Hkv, W, MK):
    """Units split over several CTAs are merged from per-CTA partials by whichever CTA arrives last, in a fixed
    order: repeated calls on the same inputs give the same bits (a stale read of another CTA's partial would not),
    and they agree with an fp32 evaluation of the step."""
    D = 128
    g = torch.Generator().manual_seed(7)
    rn = lambda *s: torch.randn(*s, generator=g)
    cnt = dev(torch.randint(0, 60, (B, Hkv, MK), generator=g).float())
    q, k, v = dev(rn(B, Hq, D).bfloat16()), dev(rn(B, Hkv, W, D).bfloat16()), dev(rn(B, Hkv, W, D).bfloat16())
    vsum = (dev(rn(B, Hkv, MK, D)) * cnt[..., None].sqrt()).bfloat16()
    cbd = dev((rn(Hkv, MK, D) * D ** -0.25).bfloat16())
    ws = api.decode_workspace(B, Hq, Hkv, D, "cuda")
    first = api.vq_attention_decode(q, q, k, k, v, cbd, cnt, vsum, workspace=ws).clone()
    differing = 0
    for _ in range(300):
        o = api.vq_attention_decode(q, q, k, k, v, cbd, cnt, vsum, workspace=ws)
        differing += int(not torch.equal(o.view(torch.int16), first.view(torch.int16)))
    torch.cuda.synchronize()
    api.check_status()
    assert differing == 0
    qf = q.float().view(B, Hkv, Hq // Hkv, D)
    s_w = torch.einsum("bhgd,bhwd->bhgw", qf, k.float()) / D ** 0.5
    s_f = (torch.einsum("bhgd,hcd->bhgc", qf, cbd.float()) / D ** 0.5).masked_fill((cnt <= 0)[:, :, None, :], float("-inf"))
    m = torch.maximum(s_w.amax(-1), s_f.amax(-1))[..., None]
    pw, pf = (s_w - m).exp(), (s_f - m).exp()
    den = pw.sum(-1) + (pf * cnt[:, :, None, :]).sum(-1)
    num = torch.einsum("bhgw,bhwd->bhgd", pw, v.float()) + torch.einsum("bhgc,bhcd->bhgd", pf, vsum.float())
    want = (num / den[..., None]).view(B, Hq, D)
    assert float((first.float() - want).abs().max()) < 2e-2     # bf16 output; observed 1e-4


def test_decode_fp16_matches_oracle(api):
    B, Hq, Hkv, D, M, K, W, L = 2, 4, 2, 128, 2, 128, 128, 640
    case = make_case(B, Hq, Hkv, L, D, M, K, W, 23, True, torch.float16)
    f = lambda t: t.float().numpy()
    cb = case["cb"].numpy()
    codes = vo.assign_codes(f(case["k3"]), cb)
    cnt, vsum = vo.build_aggregates(codes, f(case["v"]), K)
    cb16 = f(case["cb"].half())
    full = vo.attn_naive(f(case["q1"]), f(case["q2"]), f(case["k1"]), f(case["k3"]), f(case["v"]), cb16, codes, W)
    for n in (100, 300, 640):
        i = n - 1
        bd = max(0, (i - W) // 128 * 128)
        far = bd > 0
        blk = bd // 128 - 1 if far else 0
        win = lambda t: dev(t[:, :, bd:n].contiguous())
        got = api.vq_attention_decode(dev(case["q1"][:, :, i].contiguous()), dev(case["q2"][:, :, i].contiguous()),
                                      win(case["k1"]), win(case["k3"]), win(case["v"]),
                                      dev(case["cb"].reshape(Hkv, M * K, D).half()) if far else None,
                                      dev(torch.from_numpy(cnt[:, :, blk].reshape(B, Hkv, M * K).astype(np.float32))) if far else None,
                                      dev(torch.from_numpy(vsum[:, :, blk].reshape(B, Hkv, M * K, D)).half()) if far else None,
                                      n_valid=n - bd, n_bd=max(0, i - W) - bd)
        np.testing.assert_allclose(got.float().cpu().numpy(), full[:, :, i], atol=2e-2, rtol=0)


# ----------------------------------------------------------------------------- edges

def test_unused_codeword_with_a_dominating_score_is_excluded(api):
    """A codeword no key was assigned to, whose score towers over every real one: the reference masks it before
    its maximum (ops/triton_fused_vq_attn.py:44-46).  Letting it set the maximum would push every real weight
    below the exponent range and the row would come out as zeros.  The attention's copy of the codebook gets
    such a row planted (the codes and aggregates are those of the original codebook, so the row stays unused and
    the naive oracle, which only looks up the codewords of assigned codes, is unaffected)."""
    B, Hq, Hkv, L, D, M, K, W = 1, 2, 2, 768, 128, 1, 128, 128
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        case = make_case(B, Hq, Hkv, L, D, M, K, W, 41, True, dtype)
        want, _ = oracle_prefill(case)
        d = {k: dev(t) if isinstance(t, torch.Tensor) else t for k, t in case.items()}
        _, st = api.vq_attention_prefill(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], d["cb"], W, return_state=True)
        cb_act = d["cb"].reshape(Hkv, M * K, D).to(dtype).clone()
        for h in range(Hkv):
            free = (st["cnt"][0, h].sum(0) == 0).nonzero().flatten()      # unused in every block
            assert len(free) > 0
            qdir = d["q2"][0, h * (Hq // Hkv), 300:].float().mean(0)
            cb_act[h, int(free[0])] = (qdir / qdir.norm() * 2000.0).to(dtype)   # scores of hundreds of log2 units
        for impl in (("simt", "tensor") if dtype != torch.float32 else ("simt",)):
            got = api.prefill_from_aggregates(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], cb_act, st["cnt"], st["vsum"], W,
                                              impl=impl).float().cpu().numpy()
            assert np.isfinite(got).all()
            assert np.abs(got[:, :, 300:]).max() > 1e-3                # not silently zero
            assert np.abs(got - want).max() <= (1e-4 if dtype == torch.float32 else 2e-2), (dtype, impl)
    api.check_status()


def test_bounded_wait_times_out_and_the_library_keeps_working(api):
    """A wait nobody satisfies gives up after the configured number of cycles, the status word says so, and the
    next call works: nothing spins for ever, nothing traps."""
    from vqtree_b200 import native
    old = api.set_wait_limit(2_000_000)            # about one millisecond of SM clock
    try:
        api.check_status()
        api.wait_selftest()
        torch.cuda.synchronize()
        with pytest.raises(native.VqError) as e:
            api.check_status()
        assert e.value.status == -6                # VQ_ETIMEOUT
        api.check_status()                         # the word was cleared
    finally:
        assert api.set_wait_limit(old) == 2_000_000
    # a real kernel right after, with the short limit restored to the default
    case = make_case(1, 2, 2, 512, 128, 1, 128, 128, 2, True, torch.bfloat16)
    want, _ = oracle_prefill(case)
    got, _ = _run_prefill(api, case, "tensor")
    assert np.abs(got - want).max() <= 2e-2


def test_cache_advance_skips_codes_outside_the_codebook(api):
    """8-bit codes with K = 128: a code of 200 must not touch any row (canaries either side of the buffers stay
    intact) and is reported through the status word as an invalid argument."""
    from vqtree_b200 import native
    B, Hkv, D, M, K, n = 1, 2, 64, 2, 128, 96
    g = torch.Generator().manual_seed(8)
    codes = torch.randint(0, K, (B, Hkv, n, M), generator=g).to(torch.uint8)
    bad = codes.clone()
    bad[0, 1, 17, 1] = 200
    bad[0, 0, 50, 0] = 255
    v = torch.randn(B, Hkv, n, D, generator=g).bfloat16()
    pad = 4096
    def guarded(shape, dtype):
        n_el = int(np.prod(shape))
        buf = torch.full((n_el + 2 * pad,), 7.0, dtype=dtype, device="cuda")
        view = buf[pad: pad + n_el].view(shape)
        view.zero_()
        return buf, view
    bufs = [guarded((B, Hkv, M * K), torch.float32), guarded((B, Hkv, M * K, D), torch.float32), guarded((B, Hkv, M * K, D), torch.bfloat16)]
    api.check_status()
    api.cache_advance(dev(bad), dev(v), K, bufs[0][1], bufs[1][1], bufs[2][1])
    torch.cuda.synchronize()
    with pytest.raises(native.VqError) as e:
        api.check_status()
    assert e.value.status == -7
    for buf, view in bufs:
        assert bool((buf[:pad] == 7).all()) and bool((buf[-pad:] == 7).all())
    # every valid key was still folded in: equal to advancing with the two bad keys removed
    good_cnt, good_vs = torch.zeros_like(bufs[0][1]), torch.zeros_like(bufs[1][1])
    keep = torch.ones(B, Hkv, n, M, dtype=torch.bool)
    keep[0, 1, 17, 1] = False
    keep[0, 0, 50, 0] = False
    vf = v.float()
    for h in range(Hkv):
        for j in range(n):
            for m in range(M):
                if keep[0, h, j, m]:
                    r = m * K + int(codes[0, h, j, m])
                    good_cnt[0, h, r] += 1
                    good_vs[0, h, r] += vf[0, h, j].cuda()
    assert torch.equal(bufs[0][1], good_cnt)
    np.testing.assert_allclose(bufs[1][1].cpu().numpy(), good_vs.cpu().numpy(), atol=1e-5, rtol=0)
    api.check_status()


def test_strided_inputs_and_output_in_place(api):
    """[B,L,H,D] storage viewed as [B,H,L,D] for every activation and for the output: no copies needed, same
    result as the contiguous call (the layout the attention module works in, ops/attn_vq.py:207-209,442)."""
    case = make_case(2, 4, 2, 900, 128, 2, 128, 256, 51, True, torch.bfloat16)
    d = {k: dev(t) for k, t in case.items() if isinstance(t, torch.Tensor)}
    want = api.vq_attention_prefill(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], d["cb"], 256)
    blhd = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    out = torch.empty(2, 900, 4, 128, dtype=torch.bfloat16, device="cuda")
    got = api.vq_attention_prefill(blhd(d["q1"]), blhd(d["q2"]), blhd(d["k1"]), blhd(d["k3"]), blhd(d["v"]), d["cb"], 256,
                                   out=out.transpose(1, 2))
    assert got.data_ptr() == out.data_ptr()
    assert torch.equal(out.transpose(1, 2), want)
    api.check_status()


def test_prefill_sharded_equals_unsharded(api):
    """Two ranks' worth of (batch, kv-head) units, run one after the other in this process: concatenated they are
    the unsharded result bit for bit (uneven split: 3 batches x 2 kv heads over 4 ranks cuts inside a batch row)."""
    from vqtree_b200 import sharding
    case = make_case(3, 4, 2, 640, 128, 2, 128, 128, 61, True, torch.bfloat16)
    d = {k: dev(t) for k, t in case.items() if isinstance(t, torch.Tensor)}
    want = api.vq_attention_prefill(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], d["cb"], 128)
    for world in (2, 4):
        parts = [sharding.prefill_sharded(d["q1"], d["q2"], d["k1"], d["k3"], d["v"], d["cb"], 128, world, r) for r in range(world)]
        got = torch.cat(parts, 0).view(3, 2, 2, 640, 128).reshape(3, 4, 640, 128)
        assert torch.equal(got, want)
    api.check_status()
