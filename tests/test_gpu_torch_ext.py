"""torch.ops.vqattn.* against the ctypes layer: the same kernels behind both bindings, so the same bits."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from vqtree_b200 import torch_ops
    return torch_ops.load()


@pytest.fixture(scope="module")
def api():
    from vqtree_b200 import api
    return api


def _case(seed, B=2, Hq=8, Hkv=4, L=1024, D=128, M=2, K=256):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    q = rn(B, L, Hq, D).bfloat16().cuda().transpose(1, 2)          # strided views, as the projections leave them
    k = rn(B, L, Hkv, D).bfloat16().cuda().transpose(1, 2)
    v = rn(B, L, Hkv, D).bfloat16().cuda().transpose(1, 2)
    cb = (rn(Hkv, M, K, D) * D ** -0.25).cuda()
    return q, k, v, cb


def test_prefill_pipeline_through_the_dispatcher_equals_the_ctypes_path(ops, api):
    q, k, v, cb = _case(3)
    B, Hq, L, D = q.shape
    Hkv, M, K, _ = cb.shape
    W = 256
    word = api.device_status_word("cuda")
    # ctypes layer
    codes_a = api.assign_codes(k, cb)
    nb = api.far_blocks(L, W)
    cnt_a, vsum_a, sc_a, sv_a = api.build_aggregates(codes_a, v, K, nb, state_blocks=(L - W) // 128)
    cba = cb.reshape(Hkv, M * K, D).to(q.dtype)
    out_a = api.prefill_from_aggregates(q, q, k, k, v, cba, cnt_a, vsum_a, W)
    # dispatcher operators
    codes_b = torch.empty_like(codes_a)
    ws = torch.empty(ops.assign_workspace_bytes(B, Hkv, L, M, K, D), dtype=torch.uint8, device="cuda")
    ops.assign_codes(k, cb, None, codes_b, ws, word)
    cnt_b, vsum_b, sc_b, sv_b = (torch.empty_like(t) for t in (cnt_a, vsum_a, sc_a, sv_a))
    ws2 = torch.empty(ops.aggregates_workspace_bytes(B, Hkv, (L - W) // 128, M, K), dtype=torch.uint8, device="cuda")
    ops.build_aggregates(codes_b, v, K, cnt_b, vsum_b, sc_b, sv_b, (L - W) // 128, ws2, word)
    out_b = torch.empty_like(out_a)
    lse = torch.empty(B, Hq, L, device="cuda")
    ops.prefill(q, q, k, k, v, cba, cnt_b, vsum_b, W, 0.0, 0, out_b, lse, word)
    torch.cuda.synchronize()
    api.check_status()
    assert torch.equal(codes_a, codes_b)
    assert torch.equal(cnt_a, cnt_b) and torch.equal(vsum_a.view(torch.int16), vsum_b.view(torch.int16))
    assert torch.equal(sc_a, sc_b) and torch.equal(sv_a, sv_b)
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
    assert torch.isfinite(lse).all()


def test_decode_and_cache_advance_through_the_dispatcher(ops, api):
    B, Hq, Hkv, D, W, MK = 3, 24, 8, 128, 900, 512
    g = torch.Generator().manual_seed(9)
    rn = lambda *s: torch.randn(*s, generator=g).cuda()
    q, kw, vw = rn(B, Hq, D).bfloat16(), rn(B, Hkv, W, D).bfloat16(), rn(B, Hkv, W, D).bfloat16()
    cnt = torch.randint(0, 50, (B, Hkv, MK), generator=g).float().cuda()
    vsum = (rn(B, Hkv, MK, D) * cnt[..., None].sqrt()).bfloat16()
    cbd = (rn(Hkv, MK, D) * D ** -0.25).bfloat16()
    want = api.vq_attention_decode(q, q, kw, kw, vw, cbd, cnt, vsum)
    ws = torch.zeros(ops.decode_workspace_bytes(B, Hq, Hkv, D), dtype=torch.uint8, device="cuda")
    out = torch.empty_like(want)
    ops.decode(q, q, kw, kw, vw, cbd, cnt, vsum, W, 0, 0.0, ws, out, None)
    torch.cuda.synchronize()
    assert torch.equal(want.view(torch.int16), out.view(torch.int16))
    # cache advance: 128 keys folded into the aggregates
    codes = torch.randint(0, 256, (B, Hkv, 128, 2), generator=g).to(torch.uint8).cuda()
    vn = rn(B, Hkv, 128, D).bfloat16()
    c1, s1 = cnt.clone(), vsum.float()
    c2, s2 = cnt.clone(), vsum.float()
    api.cache_advance(codes, vn, 256, c1, s1, None)
    ops.cache_advance(codes, vn, 256, c2, s2, None, None)
    torch.cuda.synchronize()
    assert torch.equal(c1, c2) and torch.equal(s1, s2)


def test_errors_are_exceptions_and_the_operators_trace(ops, api):
    q, k, v, cb = _case(4, L=512)
    out = torch.empty(q.shape, dtype=q.dtype, device="cuda")
    with pytest.raises(RuntimeError, match="vqattn::prefill"):
        ops.prefill(q, q, k, k, v, None, None, None, 100, 0.0, 0, out, None, None)       # window not a multiple of 128

    def step(q, k, v, out):
        torch.ops.vqattn.prefill(q, q, k, k, v, None, None, None, 512, 0.0, 0, out, None, None)
        return out.float().sum()

    eager = step(q, k, v, out).item()
    traced = torch.compile(step, backend="eager", fullgraph=True)(q, k, v, torch.empty_like(out)).item()
    assert eager == traced
