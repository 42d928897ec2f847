"""CPU-side checks of the C ABI: the library loads, exports what the header declares, and its
argument validation answers with the documented status codes before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _native():
    from vqtree_b200 import native
    return native


def test_library_exports_every_declared_symbol():
    native = _native()
    header = (ROOT / "include" / "vqattn.h").read_text()
    declared = set(re.findall(r"\b(vqattn_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(native.EXPORTS)
    for name in declared:
        assert hasattr(native.lib, name)
    assert native.lib.vqattn_version() == int(re.search(r"#define VQATTN_VERSION (\d+)", header).group(1))


def test_struct_layout_matches_header():
    native = _native()
    # VqTensorDesc: ptr(8) dtype(4) ndim(4) shape(5*8) stride(5*8) device(4) + tail padding
    assert ctypes.sizeof(native.VqTensorDesc) == 104
    assert native.VqTensorDesc.shape.offset == 16 and native.VqTensorDesc.stride.offset == 56
    assert native.VqPrefillArgs.window.offset == 10 * 104
    assert native.VqDecodeArgs.n_valid.offset == 9 * 104


def test_aggregates_workspace_size():
    lib = _native().lib
    # per (batch, kv head, block, codebook): 128 key indices + K + 1 starts, rounded up to 16 bytes
    assert lib.vqattn_aggregates_workspace_bytes(1, 32, 247, 4, 256) == 32 * 247 * 4 * 400
    assert lib.vqattn_aggregates_workspace_bytes(2, 8, 3, 1, 512) == 2 * 8 * 3 * 656
    assert lib.vqattn_aggregates_workspace_bytes(0, 8, 3, 1, 512) == 0 and lib.vqattn_aggregates_workspace_bytes(1, 1, 1, 1, -4) == 0


def test_status_strings():
    native = _native()
    assert native.lib.vqattn_status_string(0) == b"ok"
    for code in range(-9, 0):
        assert native.lib.vqattn_status_string(code) not in (b"ok", b"unknown status")
    assert native.lib.vqattn_status_string(-99) == b"unknown status"


def test_validation_rejects_bad_arguments_without_a_device():
    native = _native()
    lib, desc = native.lib, native.desc
    k = torch.zeros(1, 2, 128, 64)
    cb = torch.zeros(2, 1, 128, 64)
    codes = torch.zeros(1, 2, 128, 1, dtype=torch.uint8)
    # null pointer
    assert lib.vqattn_assign_codes(None, desc(cb), None, desc(codes), None) == -7
    # wrong rank
    assert lib.vqattn_assign_codes(desc(k[0]), desc(cb), None, desc(codes), None) == -1
    # non-contiguous innermost dimension
    assert lib.vqattn_assign_codes(desc(k.transpose(2, 3)), desc(cb), None, desc(codes), None) == -3
    # host tensors are not on the current device (or there is no device): device error, not a crash
    assert lib.vqattn_assign_codes(desc(k), desc(cb), None, desc(codes), None) == -4
    # RoPE: null input, missing tables, no output asked for, constant position outside the tables, odd head dim
    x = torch.zeros(1, 2, 16, 64)
    tab = torch.zeros(32, 32)
    tp = ctypes.c_void_p(tab.data_ptr())
    assert lib.vqattn_rope(None, None, tp, tp, 32, 0, desc(x), None, None, None) == -7
    assert lib.vqattn_rope(desc(x), None, None, tp, 32, 0, desc(x), None, None, None) == -7
    assert lib.vqattn_rope(desc(x), None, tp, tp, 32, 0, None, None, None, None) == -7
    assert lib.vqattn_rope(desc(x), None, tp, tp, 32, 40, None, desc(x), None, None) == -7
    assert lib.vqattn_rope(desc(torch.zeros(1, 2, 16, 36)), None, tp, tp, 32, 0, desc(torch.zeros(1, 2, 16, 36)), None, None, None) == -1
    assert lib.vqattn_prefill(None, None) == -7
    assert lib.vqattn_decode(None, None) == -7
    assert lib.vqattn_decode_workspace_bytes(16, 32, 32, 128) >= 16 * 32 * 130 * 4


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    native = _native()
    monkeypatch.setattr(native, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        native._load()


def test_api_refuses_cpu_tensors():
    from vqtree_b200 import api
    with pytest.raises(ValueError):
        api.assign_codes(torch.zeros(1, 1, 128, 64), torch.zeros(1, 1, 128, 64))
