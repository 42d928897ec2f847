"""Mirror of the reference's ``ops/mini_vq.py`` on the CUDA library."""
from __future__ import annotations

import torch

from . import api


def multi_head_single_quantize(inp: torch.Tensor, codebook: torch.Tensor):
    """Same contract as ops/mini_vq.py:4-18.

    inp [B,H,L,D], codebook [H,C,D] -> (quantized [B,H,L,D], ids [B,H,L] int64, onehot [B,H,L,C] int64).
    The arg-max of the inner products runs in ``vqattn_assign_codes``; the reconstruction and the
    one-hot tensor are pure index plumbing on the result.
    """
    bsz, head, seqlen, hsz = inp.shape
    assert codebook.shape[0] == head and codebook.shape[2] == hsz
    k = inp if inp.dtype in (torch.float32, torch.bfloat16, torch.float16) else inp.float()
    ids = api.assign_codes(k, codebook[:, None].float().contiguous(), out_dtype=torch.int64)[..., 0]
    quantized = torch.gather(codebook[None].expand(bsz, -1, -1, -1), 2, ids[..., None].expand(-1, -1, -1, hsz))
    onehot = torch.nn.functional.one_hot(ids, codebook.shape[1])
    return quantized, ids, onehot
