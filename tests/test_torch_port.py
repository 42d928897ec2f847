"""The PyTorch CPU port (the timed CPU baseline) against the C oracle and the reference's golden output."""
import numpy as np
import torch

from oracle import torch_port as tp
from oracle import vq_oracle as vo
from tests.vq_cases import make_case


def test_port_matches_oracle_multi_codebook():
    case = make_case(1, 4, 2, 640, 64, 2, 128, 128, 12, True)
    codes = tp.quantize(case["k3"], case["cb"])
    want_codes = vo.assign_codes(case["k3"].numpy(), case["cb"].numpy())
    mism = codes.numpy() != want_codes
    assert mism.mean() < 1e-3  # BLAS summation order may flip a near tie
    out = tp.naive_attention(case["q1"], case["q2"], case["k1"], case["k3"], case["v"], case["cb"],
                             torch.from_numpy(want_codes), case["W"])
    want = vo.attn_naive(*(case[n].numpy() for n in ("q1", "q2", "k1", "k3", "v")), case["cb"].numpy(), want_codes, case["W"])
    np.testing.assert_allclose(out.numpy(), want, atol=2e-5, rtol=0)


def test_port_matches_reference_golden(golden_dir):
    gd = np.load(golden_dir / "naive_selftest.npz")
    W = int(gd["window"])
    q, k, v, cb = (torch.from_numpy(gd[n]) for n in ("q", "k", "v", "codebook"))
    L, D = q.shape[2], q.shape[3]
    cos, sin = vo.rope_tables(max(L, W + 2), D)
    pos = np.arange(L)
    q1 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, pos))
    k1 = torch.from_numpy(vo.apply_rope(k.numpy(), cos, sin, pos))
    q2 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, np.full(L, W + 1)))
    out = tp.prefill(q1, q2, k1, k, v, cb[:, None], W)
    np.testing.assert_allclose(out.numpy(), gd["out"], atol=3e-5, rtol=0)
