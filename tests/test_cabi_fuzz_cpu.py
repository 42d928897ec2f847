"""Shape / stride / dtype fuzzing of the C ABI's argument validation on the host.

No device is touched: every call here is malformed in some way or describes host memory, so the library must
answer with a negative status - never crash, never launch.  (hypothesis drives the descriptors.)"""
import ctypes

import pytest
import torch
from hypothesis import given, settings, strategies as st

native = pytest.importorskip("vqtree_b200.native")


def _desc(ndim, shape, stride, dtype, ptr):
    d = native.VqTensorDesc()
    d.ptr, d.dtype, d.ndim, d.device = ptr, dtype, ndim, 0
    for i in range(5):
        d.shape[i], d.stride[i] = shape[i], stride[i]
    return d


dims = st.integers(min_value=-2, max_value=7)
sizes = st.lists(st.integers(min_value=-3, max_value=4096), min_size=5, max_size=5)
strides = st.lists(st.integers(min_value=-8, max_value=1 << 20), min_size=5, max_size=5)
dtypes = st.integers(min_value=-1, max_value=9)
descs = st.builds(_desc, dims, sizes, strides, dtypes, st.sampled_from([None, 4096]))


@settings(max_examples=150, deadline=None)
@given(descs, descs, descs, descs)
def test_assign_and_aggregates_reject_arbitrary_descriptors(a, b, c, d):
    lib = native.lib
    P = ctypes.byref
    assert lib.vqattn_assign_codes(P(a), P(b), P(c), P(d), None) < 0
    assert lib.vqattn_assign_codes_ws(P(a), P(b), None, P(d), None, 0, None, None) < 0
    assert lib.vqattn_build_aggregates(P(a), P(b), 256, P(c), P(d), None) < 0
    assert lib.vqattn_build_aggregates_ws(P(a), P(b), 256, P(c), P(d), None, 0, None, None) < 0
    assert lib.vqattn_build_aggregates_state(P(a), P(b), 256, P(c), P(d), P(c), P(d), 1, None, 0, None, None) < 0
    assert lib.vqattn_build_aggregates_state(P(a), P(b), 256, P(c), P(d), None, None, 1, None, 0, None, None) < 0
    assert lib.vqattn_gather_aggregates(P(a), P(b), P(c), P(d), None) < 0
    assert lib.vqattn_cache_advance(P(a), P(b), 128, P(c), P(d), None, None, None) < 0


@settings(max_examples=100, deadline=None)
@given(st.lists(descs, min_size=10, max_size=10), st.integers(-256, 4096), st.integers(-1, 5))
def test_prefill_and_decode_reject_arbitrary_descriptors(ds, window, impl):
    lib = native.lib
    a = native.VqPrefillArgs()
    for name, d in zip(("q1", "q2", "k1", "k3", "v", "codebook", "cnt", "vsum", "out", "lse2"), ds):
        setattr(a, name, d)
    a.window, a.impl = window, impl
    assert lib.vqattn_prefill(ctypes.byref(a), None) < 0
    b = native.VqDecodeArgs()
    for name, d in zip(("q1", "q2", "k1_win", "k3_win", "v_win", "codebook", "cnt", "vsum", "out"), ds):
        setattr(b, name, d)
    b.n_valid, b.n_bd, b.use_far = window, impl, 1
    assert lib.vqattn_decode(ctypes.byref(b), None) < 0
    assert lib.vqattn_decode_static(ctypes.byref(b), None) < 0
    s = native.VqDecodeStepArgs()
    s.decode = b
    s.q, s.k, s.v, s.q1, s.q2 = ds[0], ds[1], ds[2], ds[3], ds[4]
    assert lib.vqattn_decode_step(ctypes.byref(s), None) < 0


def test_well_formed_host_tensors_are_refused_as_not_on_the_device():
    lib, desc = native.lib, native.desc
    k, cb, codes = torch.zeros(1, 2, 128, 64), torch.zeros(2, 1, 128, 64), torch.zeros(1, 2, 128, 1, dtype=torch.uint8)
    P = ctypes.byref
    assert lib.vqattn_assign_codes(P(desc(k)), P(desc(cb)), None, P(desc(codes)), None) == -4
    assert lib.vqattn_status_from_word(0) == 0 and lib.vqattn_status_from_word(1) == -6
    assert lib.vqattn_status_from_word(2) == -7 and lib.vqattn_status_from_word(3) == -7
    assert lib.vqattn_wait_selftest(None, None) == -7
    old = lib.vqattn_set_wait_limit_cycles(12345)
    assert lib.vqattn_set_wait_limit_cycles(old) == 12345
