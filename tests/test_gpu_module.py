"""The attention module, its cache and the transformers integration on the real kernels (the scenarios of
tests/module_scenarios.py; the CPU suite runs them on a test double)."""
import pytest
import torch

from tests import module_scenarios as ms

pytestmark = pytest.mark.gpu


def test_reference_selftest_replay_fp16_then_300_tokens():
    """ops/attn_vq.py:534-556 - LlamaConfig(hidden_size=128, 2 heads), fp16, LEN 511, window 256, codebook
    randn(2,128,64) - with an assertion (2e-2, the reference's half-precision tolerance), then 300 generated
    tokens through the same module and cache object."""
    err, worst = ms.selftest_replay("cuda", torch.float16, 2e-2, LEN=511, W=256, C=128, n_decode=300)
    print(f"fp16 self-test: prefill max-abs {err:.2e}, decode max-abs {worst:.2e}")
    from vqtree_b200 import api
    api.check_status()


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
def test_selftest_replay_other_dtypes(dtype, tol):
    ms.selftest_replay("cuda", dtype, tol, LEN=511, W=256, C=128, n_decode=150)
    ms.selftest_replay("cuda", dtype, tol, LEN=640, W=128, C=128, n_decode=140, M=2, seed=9)


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-2), (torch.float32, 1e-4)])
def test_short_prefill_is_plain_causal(dtype, tol):
    ms.short_prefill_is_plain_causal("cuda", dtype, tol, W=128, L=200)
    ms.short_prefill_is_plain_causal("cuda", dtype, tol, W=128, L=256)


def test_save_load_continues(tmp_path):
    ms.save_load_continues("cuda", torch.bfloat16, tmp_path)


def test_tiny_llama_generate_under_use_rerope():
    ms.tiny_llama_generate("cuda", torch.float32, 2e-3, n_new=40, L=400)
    ms.tiny_llama_generate("cuda", torch.bfloat16, 0.25, n_new=24, L=300)
