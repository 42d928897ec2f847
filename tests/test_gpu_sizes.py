"""Parity at the benchmark configurations' real sizes (sampled rows against the naive oracle).

Shapes: config 2 (B1 H32 L8192 W1024 M4 K256, RoPE), config 4 (B2 H32 L16384 W512 M4 K512, ReRoPE), the 32K
headline point (config 2 at L = 32768), a config-5-shaped case (B2 Hq32/Hkv8 W2048 M8 K256, L = 16384) and
config 3's decode step (B16 H32 MK1024 W1024, context 32768).  Codes: the tensor-core assignment against the
exact kernel on ALL keys and against the oracle on sampled key ranges; aggregates against the oracle for one
unit; attention rows against the naive oracle (tolerance 2e-2 in bf16: the reference's own half-precision
tolerance, ops/triton_fused_local_attn.py:283)."""
import numpy as np
import pytest
import torch

from oracle import sampled, vq_oracle as vo

pytestmark = pytest.mark.gpu

CASES = {
    "c2": dict(B=1, Hq=32, Hkv=32, D=128, L=8192, W=1024, M=4, K=256, rerope=False, seed=1),
    "c4": dict(B=2, Hq=32, Hkv=32, D=128, L=16384, W=512, M=4, K=512, rerope=True, seed=3),
    "c2_32k": dict(B=1, Hq=32, Hkv=32, D=128, L=32768, W=1024, M=4, K=256, rerope=False, seed=1),
    "c5_16k": dict(B=2, Hq=32, Hkv=8, D=128, L=16384, W=2048, M=8, K=256, rerope=False, seed=4),
}


@pytest.mark.parametrize("name", list(CASES))
def test_prefill_path_at_benchmark_size(name):
    import bench
    from vqtree_b200 import api
    w = CASES[name]
    dev = torch.device("cuda")
    q1, q2, k1, k3, v, cb = bench.make_inputs(w, dev)
    B, Hkv, L, W, M, K, D = w["B"], w["Hkv"], w["L"], w["W"], w["M"], w["K"], w["D"]
    # ---- codes: tensor-core path == exact kernel on every key; == oracle on sampled ranges
    codes = api.assign_codes(k3, cb)
    exact = api.assign_codes(k3, cb, impl="simt")
    assert torch.equal(codes, exact), f"{int((codes != exact).sum())} codes differ between the two kernels"
    units = [(0, 0), (B - 1, Hkv // 2), (B - 1, Hkv - 1)]
    kr = [(0, 256), (L // 2 - 100, L // 2 + 156), (L - 256, L)]
    assert sampled.codes_equal_on_ranges(codes, k3, cb, units, kr)
    # ---- aggregates: one unit against the oracle, first / middle / last block bit for bit
    nb = api.far_blocks(L, W)
    cnt, vsum = api.build_aggregates(codes, v, K, nb)
    b, h = units[1]
    cw, vw = vo.build_aggregates(codes[b:b + 1, h:h + 1].cpu().to(torch.int32).numpy(), v[b:b + 1, h:h + 1].float().cpu().numpy(), K, NB=nb)
    for blk in (0, nb // 2, nb - 1):
        np.testing.assert_array_equal(cnt[b, h, blk].cpu().numpy(), cw[0, 0, blk].reshape(-1).astype(np.float32))
        np.testing.assert_array_equal(vsum[b, h, blk].float().cpu().numpy(), vo.round_bf16(vw[0, 0, blk].reshape(M * K, D)))
    del cw, vw
    # ---- attention rows
    cb_act = cb.reshape(Hkv, M * K, D).to(torch.bfloat16)
    out = api.prefill_from_aggregates(q1, q2, k1, k3, v, cb_act, cnt, vsum, W)
    torch.cuda.synchronize()
    api.check_status()
    assert torch.isfinite(out.float()).all()
    err, rows = sampled.prefill_rows_max_err(out, q1, q2, k1, k3, v, cb_act.float().reshape(Hkv, M, K, D), codes, W, units,
                                             sampled.row_ranges(L, W, seed=w["seed"]))
    assert rows >= 20 and err <= 2e-2, f"{name}: max-abs {err} over {rows} rows"


@pytest.mark.parametrize("cb_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n_valid,n_bd", [(1024, 0), (1152, 127)])
def test_decode_at_config3_size(cb_dtype, n_valid, n_bd):
    """B16 H32 D128 M4xK256 W1024: the benchmarked call (1024 window rows) and the true step at context 32768
    (1152 rows of which the first 127 are scored with the constant-position query)."""
    from vqtree_b200 import api
    B, H, D, MK, Nwin = 16, 32, 128, 1024, 1152
    g = torch.Generator(device="cuda").manual_seed(2)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    q1, q2 = rn(B, H, D).bfloat16(), rn(B, H, D).bfloat16()
    k1, k3, v = (rn(B, H, Nwin, D).bfloat16() for _ in range(3))
    cnt = torch.randint(0, 60, (B, H, MK), generator=g, device="cuda").float()
    cnt[:, :, ::7] = 0                                   # codes without members
    vsum = (rn(B, H, MK, D) * cnt[..., None].sqrt()).bfloat16()
    cb = (rn(H, MK, D) * D ** -0.25).to(cb_dtype)
    got = api.vq_attention_decode(q1, q2, k1, k3, v, cb, cnt, vsum, n_valid=n_valid, n_bd=n_bd)
    torch.cuda.synchronize()
    api.check_status()
    f = lambda t: t.float().cpu().numpy()
    want = vo.decode(f(q1), f(q2), f(k1), f(k3), f(v), f(cb).reshape(H, 1, MK, D), f(cnt).reshape(B, H, 1, MK),
                     f(vsum).reshape(B, H, 1, MK, D), n_valid, n_bd)
    np.testing.assert_allclose(f(got), want, atol=2e-2, rtol=0)
