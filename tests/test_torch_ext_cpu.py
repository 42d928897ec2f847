"""The PyTorch C++ extension over the C ABI (torch.ops.vqattn.*): loading, schemas, sizes - no GPU needed."""
import re
from pathlib import Path

import pytest
import torch

from vqtree_b200 import native, torch_ops


@pytest.fixture(scope="module")
def ops():
    return torch_ops.load()


def test_extension_loads_and_reports_the_header_version(ops):
    header = (Path(__file__).resolve().parents[1] / "include" / "vqattn.h").read_text()
    assert int(ops.abi_version()) == int(re.search(r"#define VQATTN_VERSION (\d+)", header).group(1))


def test_workspace_sizes_equal_the_c_abi(ops):
    lib = native.lib
    assert ops.assign_workspace_bytes(1, 32, 32768, 4, 256, 128) == lib.vqattn_assign_workspace_bytes(1, 32, 32768, 4, 256, 128)
    assert ops.aggregates_workspace_bytes(2, 8, 3, 1, 512) == lib.vqattn_aggregates_workspace_bytes(2, 8, 3, 1, 512)
    assert ops.decode_workspace_bytes(16, 32, 32, 128) == lib.vqattn_decode_workspace_bytes(16, 32, 32, 128)


def test_operators_are_registered_as_out_variants(ops):
    for name in ("assign_codes", "build_aggregates", "prefill", "decode", "cache_advance"):
        schema = str(getattr(torch.ops.vqattn, name).default._schema)
        assert "-> ()" in schema and "(a!)" in schema, schema       # writes into its arguments, returns nothing


def test_there_is_no_cpu_kernel(ops):
    q = torch.zeros(1, 1, 128, 64)
    with pytest.raises(NotImplementedError):
        ops.prefill(q, q, q, q, q, None, None, None, 128, 0.0, 0, q.clone(), None, None)
    with pytest.raises(NotImplementedError):
        ops.assign_codes(q, torch.zeros(1, 1, 128, 64), None, torch.zeros(1, 1, 128, 1, dtype=torch.uint8), None, None)
