"""Host logic of the attention module, the cache and the file formats, on CPU.

The kernels are replaced by the oracle-backed test double (tests/fake_backend.py); what is tested here is
everything above the C ABI: projections and layouts, dispatch, the window / boundary bookkeeping of the
cache across block moves, save / load, the transformers integration.  tests/test_gpu_module.py runs the
same scenarios on the real kernels."""
import pickle

import numpy as np
import pytest
import torch

from tests import fake_backend, module_scenarios as ms
from vqtree_b200 import codebook_io
from vqtree_b200.attn_vq import BLOCK_SIZE, AttentionMode, VectorQuantizedReRoPECache, use_rerope


@pytest.fixture(autouse=True)
def _fake_kernels():
    with fake_backend.installed():
        yield


def test_selftest_replay_and_decode_across_boundaries():
    # the reference's self-test shape, shortened decode (the oracle-backed double is slow); fp32
    ms.selftest_replay("cpu", torch.float32, 1e-4, LEN=511, W=256, n_decode=140)


def test_selftest_replay_additive_codebooks():
    ms.selftest_replay("cpu", torch.float32, 1e-4, LEN=400, W=128, C=128, n_decode=40, M=2)


def test_short_prefill_is_plain_causal():
    ms.short_prefill_is_plain_causal("cpu", torch.float32, 1e-4)


def test_save_load_continues(tmp_path):
    ms.save_load_continues("cpu", torch.float32, tmp_path, LEN=300, W=128, n_decode=30)


def test_tiny_llama_generate():
    ms.tiny_llama_generate("cpu", torch.float32, 1e-3, n_new=12, L=300)


def test_cache_interface_and_errors():
    cb = torch.zeros(2, 128, 64)
    c = VectorQuantizedReRoPECache(256, cb, attention_mode=AttentionMode.SORT_BASED_LINEAR)
    assert BLOCK_SIZE == 128 and c.window_length == 256 and c.seen_tokens == 0
    assert c.get_seq_length(0) == 0 and c.get_usable_length(5, 0) == 0 and c.get_max_length() == int(1e8)
    with pytest.raises(AssertionError):
        VectorQuantizedReRoPECache(100, cb)                  # window not a multiple of the block
    with pytest.raises(AssertionError):
        VectorQuantizedReRoPECache(128, torch.zeros(2, 100, 64))   # codebook size % 128 (ops/attn_vq.py:45)
    k = torch.zeros(1, 2, 10, 64)
    c.update_prefill(torch.zeros(1, 2, 128), torch.zeros(1, 2, 128, 64), k, k, 0, 10, {"key_unrotated": k})
    assert c.get_seq_length(0) == 10 and c.get_usable_length(1, 0) == 10 and c.seen_tokens == 10
    with pytest.raises(RuntimeError, match="prefilling twice"):  # ops/attn_vq.py:126
        c.update_prefill(torch.zeros(1, 2, 128), torch.zeros(1, 2, 128, 64), k, k, 0, 10, {"key_unrotated": k})
    module = ms.make_module(torch.float32, "cpu")
    with pytest.raises(AssertionError, match="VQReRoPECache is required"):
        module(hidden_states=torch.zeros(1, 4, 128), past_key_value=None)
    with pytest.raises(AssertionError, match="Only support prefilling or generation"):
        module(hidden_states=torch.zeros(1, 4, 128), past_key_value=c)
    bad = VectorQuantizedReRoPECache(128, cb, attention_mode="nonsense")
    with pytest.raises(KeyError, match="Bad attention mode"):
        module(hidden_states=torch.zeros(1, 300, 128), past_key_value=bad)


def test_use_rerope_restores_the_class():
    from transformers.models.llama import modeling_llama as ml
    before = getattr(ml, "LLAMA_ATTENTION_CLASSES", {}).get("flash_attention_2", ml.LlamaAttention)
    with use_rerope():
        inside = getattr(ml, "LLAMA_ATTENTION_CLASSES", {}).get("flash_attention_2", ml.LlamaAttention)
        assert inside.__name__ == "LlamaFlashAttention2VectorQuantizedReRoPE"
    after = getattr(ml, "LLAMA_ATTENTION_CLASSES", {}).get("flash_attention_2", ml.LlamaAttention)
    assert after is before


def test_codebook_pickle_roundtrip_and_errors(tmp_path):
    # the structure build_quantizer/120_build_additive_quantizer.py:60-66 writes: {(layer, head): [M arrays [K, D]]}
    rng = np.random.default_rng(0)
    raw = {(l, h): [rng.standard_normal((512, 16)).astype(np.float32) for _ in range(4)] for l in range(3) for h in range(2)}
    with open(tmp_path / "cb.pkl", "wb") as f:
        pickle.dump(raw, f)
    got = codebook_io.load_codebooks(tmp_path / "cb.pkl")
    assert sorted(got) == [0, 1, 2] and got[0].shape == (2, 4, 512, 16) and got[0].dtype == torch.float32
    np.testing.assert_array_equal(got[1][1, 2].numpy(), raw[(1, 1)][2])
    codebook_io.save_codebooks(got, tmp_path / "again.pkl")
    with open(tmp_path / "again.pkl", "rb") as f:
        again = pickle.load(f)
    assert sorted(again) == sorted(raw) and all(np.array_equal(again[k][m], raw[k][m]) for k in raw for m in range(4))
    del raw[(1, 0)]
    with open(tmp_path / "hole.pkl", "wb") as f:
        pickle.dump(raw, f)
    with pytest.raises(ValueError, match="missing"):
        codebook_io.load_codebooks(tmp_path / "hole.pkl")
    with open(tmp_path / "evil.pkl", "wb") as f:
        pickle.dump({(0, 0): [print]}, f)
    with pytest.raises(pickle.UnpicklingError):
        codebook_io.load_codebooks(tmp_path / "evil.pkl")
