"""The workspace-free decode entry point against the regular one.

``vqattn_decode_static`` exists for hosts that cannot give the library a workspace buffer (a server
that has already handed all spare HBM to its KV-cache pool, a runtime that forbids device allocation
inside the serving step): its split/merge scratch is a fixed array inside the library.  It must return
what ``vqattn_decode`` returns, call after call, although every call reuses the same scratch bytes.
This file is collected last so that a failure here cannot hide any other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, Hkv, D, Nwin, MK, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    cnt = torch.randint(0, 40, (B, Hkv, MK), generator=g).float()
    return dict(q1=r(B, Hq, D).to(dtype).cuda(), q2=r(B, Hq, D).to(dtype).cuda(),
                k1=r(B, Hkv, Nwin, D).to(dtype).cuda(), k3=r(B, Hkv, Nwin, D).to(dtype).cuda(),
                v=r(B, Hkv, Nwin, D).to(dtype).cuda(), cb=(r(Hkv, MK, D) * D ** -0.25).cuda(),
                cnt=cnt.cuda(), vsum=(r(B, Hkv, MK, D) * cnt[..., None].sqrt()).to(dtype).cuda())


def _run(api, c, n_valid, n_bd, static):
    out = torch.empty_like(c["q1"])
    api.vq_attention_decode(c["q1"], c["q2"], c["k1"], c["k3"], c["v"], c["cb"], c["cnt"], c["vsum"], n_valid=n_valid,
                            n_bd=n_bd, out=out, static_scratch=static)
    torch.cuda.synchronize()
    api.check_status()
    return out.float().cpu().numpy()


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    from vqtree_b200 import api, native
    assert native.lib.vqattn_decode_static_capacity() == 16 << 20
    # two different problems back to back: the second call finds the first call's bytes in the scratch
    a = _case(1, 4, 8, 8, 128, 700, 512)
    b = _case(2, 2, 8, 2, 128, 384, 256)      # GQA group of 4, other split layout
    for c, n_valid, n_bd in ((a, 650, 37), (b, 384, 0), (a, 700, 128)):
        want = _run(api, c, n_valid, n_bd, static=False)
        got = _run(api, c, n_valid, n_bd, static=True)
        np.testing.assert_allclose(got, want, atol=2e-2, rtol=0)
        got2 = _run(api, c, n_valid, n_bd, static=True)
        np.testing.assert_array_equal(got2, got)


def test_static_scratch_rejects_what_does_not_fit():
    from vqtree_b200 import api, native
    B, Hq = 64, 128                            # the workspace bound for this shape exceeds 16 MiB
    assert native.lib.vqattn_decode_workspace_bytes(B, Hq, Hq, 128) > native.lib.vqattn_decode_static_capacity()
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(native.VqError) as e:
        api.vq_attention_decode(z(B, Hq, 128), z(B, Hq, 128), z(B, Hq, 64, 128), z(B, Hq, 64, 128), z(B, Hq, 64, 128),
                                None, None, None, out=z(B, Hq, 128), static_scratch=True)
    assert e.value.status == -9
