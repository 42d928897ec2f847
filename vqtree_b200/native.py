"""ctypes binding of the C ABI declared in ``include/vqattn.h``.

The library is the product: if ``libvqattn.so`` is missing or a symbol cannot be resolved this
module raises at import time - there is no fallback implementation.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libvqattn.so"

MAX_DIMS = 5
BLOCK = 128

VQ_F32, VQ_BF16, VQ_U8, VQ_U16, VQ_I32, VQ_I64, VQ_F16 = range(7)
WORD_TIMEOUT, WORD_BAD_POSITION, WORD_BAD_CODE = 1, 2, 3
IMPL_AUTO, IMPL_SIMT, IMPL_TENSOR = 0, 1, 2

_DTYPES = {
    torch.float32: VQ_F32,
    torch.bfloat16: VQ_BF16,
    torch.float16: VQ_F16,
    torch.uint8: VQ_U8,
    torch.uint16: VQ_U16,
    torch.int32: VQ_I32,
    torch.int64: VQ_I64,
}

EXPORTS = (
    "vqattn_version", "vqattn_status_string", "vqattn_assign_codes", "vqattn_build_aggregates",
    "vqattn_aggregates_workspace_bytes", "vqattn_build_aggregates_ws", "vqattn_build_aggregates_state",
    "vqattn_gather_aggregates", "vqattn_prefill", "vqattn_decode_workspace_bytes", "vqattn_decode",
    "vqattn_cache_advance", "vqattn_decode_static_capacity", "vqattn_decode_static",
    "vqattn_assign_workspace_bytes", "vqattn_assign_codes_ws", "vqattn_rope",
    "vqattn_status_from_word", "vqattn_set_wait_limit_cycles", "vqattn_wait_selftest", "vqattn_rope_qk",
    "vqattn_decode_append", "vqattn_decode_step",
)


class VqTensorDesc(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.c_int64 * MAX_DIMS),
        ("stride", ctypes.c_int64 * MAX_DIMS),
        ("device", ctypes.c_int32),
    ]


class VqPrefillArgs(ctypes.Structure):
    _fields_ = [(n, VqTensorDesc) for n in ("q1", "q2", "k1", "k3", "v", "codebook", "cnt", "vsum", "out", "lse2")] + [
        ("window", ctypes.c_int64),
        ("scale", ctypes.c_float),
        ("impl", ctypes.c_int32),
        ("status_word", ctypes.c_void_p),
    ]


class VqDecodeArgs(ctypes.Structure):
    _fields_ = [(n, VqTensorDesc) for n in ("q1", "q2", "k1_win", "k3_win", "v_win", "codebook", "cnt", "vsum", "out")] + [
        ("n_valid", ctypes.c_int64),
        ("n_bd", ctypes.c_int64),
        ("use_far", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("status_word", ctypes.c_void_p),
    ]


class VqDecodeStepArgs(ctypes.Structure):
    _fields_ = [("q", VqTensorDesc), ("k", VqTensorDesc), ("v", VqTensorDesc), ("positions", ctypes.c_void_p),
                ("pos", ctypes.c_int64), ("cos_tab", ctypes.c_void_p), ("sin_tab", ctypes.c_void_p), ("n_pos", ctypes.c_int64),
                ("const_pos", ctypes.c_int64), ("q1", VqTensorDesc), ("q2", VqTensorDesc), ("row", ctypes.c_int64),
                ("decode", VqDecodeArgs)]


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m vqtree_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback for this path")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name in EXPORTS:
        getattr(lib, name)  # raises AttributeError on a missing export
    P = ctypes.POINTER
    lib.vqattn_version.restype = ctypes.c_int
    lib.vqattn_status_string.restype = ctypes.c_char_p
    lib.vqattn_status_string.argtypes = [ctypes.c_int]
    lib.vqattn_assign_codes.argtypes = [P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p]
    lib.vqattn_assign_workspace_bytes.restype = ctypes.c_size_t
    lib.vqattn_assign_workspace_bytes.argtypes = [ctypes.c_int64] * 6
    lib.vqattn_assign_codes_ws.argtypes = [P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p,
                                           ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_build_aggregates.argtypes = [P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int32, P(VqTensorDesc),
                                            P(VqTensorDesc), ctypes.c_void_p]
    lib.vqattn_aggregates_workspace_bytes.restype = ctypes.c_size_t
    lib.vqattn_aggregates_workspace_bytes.argtypes = [ctypes.c_int64] * 5
    lib.vqattn_build_aggregates_ws.argtypes = [P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int32, P(VqTensorDesc), P(VqTensorDesc),
                                               ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_build_aggregates_state.argtypes = [P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int32, P(VqTensorDesc), P(VqTensorDesc),
                                                  P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t,
                                                  ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_gather_aggregates.argtypes = [P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p]
    lib.vqattn_prefill.argtypes = [P(VqPrefillArgs), ctypes.c_void_p]
    lib.vqattn_decode_workspace_bytes.restype = ctypes.c_size_t
    lib.vqattn_decode_workspace_bytes.argtypes = [ctypes.c_int64] * 4
    lib.vqattn_decode.argtypes = [P(VqDecodeArgs), ctypes.c_void_p]
    lib.vqattn_decode_static.argtypes = [P(VqDecodeArgs), ctypes.c_void_p]
    lib.vqattn_decode_static_capacity.restype = ctypes.c_size_t
    lib.vqattn_cache_advance.argtypes = [P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int32, P(VqTensorDesc),
                                         P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_rope_qk.argtypes = [P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_int64, ctypes.c_int64, P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc),
                                   ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_decode_append.argtypes = [P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, P(VqTensorDesc),
                                         P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), P(VqTensorDesc), ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_decode_step.argtypes = [P(VqDecodeStepArgs), ctypes.c_void_p]
    lib.vqattn_status_from_word.argtypes = [ctypes.c_int32]
    lib.vqattn_set_wait_limit_cycles.argtypes = [ctypes.c_int64]
    lib.vqattn_set_wait_limit_cycles.restype = ctypes.c_int64
    lib.vqattn_wait_selftest.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.vqattn_rope.argtypes = [P(VqTensorDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                P(VqTensorDesc), P(VqTensorDesc), ctypes.c_void_p, ctypes.c_void_p]
    for name in EXPORTS:
        if name not in ("vqattn_status_string", "vqattn_decode_workspace_bytes", "vqattn_decode_static_capacity",
                        "vqattn_assign_workspace_bytes", "vqattn_aggregates_workspace_bytes", "vqattn_set_wait_limit_cycles"):
            getattr(lib, name).restype = ctypes.c_int
    return lib


lib = _load()


class VqError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {lib.vqattn_status_string(status).decode()} (status {status})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise VqError(status, where)


def desc(t: torch.Tensor | None, d: VqTensorDesc | None = None) -> VqTensorDesc:
    """Describe a tensor for the C ABI (None -> a descriptor with a NULL pointer); ``d``: a descriptor to refill."""
    if d is None:
        d = VqTensorDesc()
    if t is None:
        d.ptr = None
        return d
    if t.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {t.dtype}")
    if t.dim() > MAX_DIMS:
        raise ValueError("too many dimensions")
    d.ptr = t.data_ptr()
    d.dtype = _DTYPES[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    d.device = t.device.index if t.is_cuda else -1
    return d


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device) -> int:
    """Handle of torch's current stream on ``device`` (the per-token decode path calls this once per step: the raw
    query avoids building a Stream object)."""
    if _RAW_STREAM is not None:
        idx = device if isinstance(device, int) else torch.device(device).index
        if idx is not None:
            return _RAW_STREAM(idx)
    return torch.cuda.current_stream(device).cuda_stream
