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


def _case(seed, B, Hq, Hkv, D, Nwin, MK, dtype=torch.bfloat16, cb_dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    cnt = torch.randint(0, 40, (B, Hkv, MK), generator=g).float()
    return dict(q1=r(B, Hq, D).to(dtype).cuda(), q2=r(B, Hq, D).to(dtype).cuda(),
                k1=r(B, Hkv, Nwin, D).to(dtype).cuda(), k3=r(B, Hkv, Nwin, D).to(dtype).cuda(),
                v=r(B, Hkv, Nwin, D).to(dtype).cuda(), cb=(r(Hkv, MK, D) * D ** -0.25).to(cb_dtype).cuda(),
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
    c16 = _case(3, 3, 8, 4, 128, 512, 256, cb_dtype=torch.bfloat16)   # 16-bit codebook: the tensor-core decode kernel
    d64 = _case(4, 2, 4, 4, 64, 300, 128)                              # head dim 64
    f32 = _case(5, 2, 4, 2, 128, 260, 128, dtype=torch.float32)        # fp32 caches: the register-streaming kernel
    for c, n_valid, n_bd in ((a, 650, 37), (b, 384, 0), (a, 700, 128), (c16, 500, 100), (d64, 300, 5), (f32, 260, 0)):
        want = _run(api, c, n_valid, n_bd, static=False)
        got = _run(api, c, n_valid, n_bd, static=True)
        np.testing.assert_allclose(got, want, atol=2e-2, rtol=0)
        got2 = _run(api, c, n_valid, n_bd, static=True)
        np.testing.assert_array_equal(got2, got)


def test_static_scratch_call_allocates_nothing():
    """Neither the caching allocator of torch nor the driver hands out memory during the call: the bytes torch
    holds and the free bytes of the device are the same before and after (output preallocated, one warm-up
    call first so that the library's one-time set-up on this device is over)."""
    from vqtree_b200 import api
    c = _case(6, 4, 8, 8, 128, 640, 512)
    out = torch.empty_like(c["q1"])
    call = lambda: api.vq_attention_decode(c["q1"], c["q2"], c["k1"], c["k3"], c["v"], c["cb"], c["cnt"], c["vsum"],
                                           n_valid=640, n_bd=3, out=out, static_scratch=True)
    call()
    torch.cuda.synchronize()
    held, reserved, free = torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0]
    call()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held and torch.cuda.memory_reserved() == reserved
    assert torch.cuda.mem_get_info()[0] == free


def test_static_scratch_rejects_what_does_not_fit():
    from vqtree_b200 import api, native
    B, Hq = 64, 128                            # the workspace bound for this shape exceeds 16 MiB
    assert native.lib.vqattn_decode_workspace_bytes(B, Hq, Hq, 128) > native.lib.vqattn_decode_static_capacity()
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(native.VqError) as e:
        api.vq_attention_decode(z(B, Hq, 128), z(B, Hq, 128), z(B, Hq, 64, 128), z(B, Hq, 64, 128), z(B, Hq, 64, 128),
                                None, None, None, out=z(B, Hq, 128), static_scratch=True)
    assert e.value.status == -9
