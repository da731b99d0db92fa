"""Small host-side helpers (mirrors of nunchaku/utils.py:77-93 where they exist)."""
from __future__ import annotations

import contextlib
import os

import torch

from . import _lib


def ceil_divide(x: int, divisor: int) -> int:
    """nunchaku/utils.py:77-93."""
    return (x + divisor - 1) // divisor


_layout_env: tuple[str | None, int] | None = None


def default_act_layout() -> int:
    """Memory order of the activation-side tensors handed from the quantiser to the GEMM.

    ``native`` (default) is what the sm_100a GEMM streams with TMA; ``reference`` is the
    reference's mma.sync fragment order (set ``SVDQ_B200_ACT_LAYOUT=reference``), which the
    GEMM converts back before use.
    """
    global _layout_env
    raw = os.environ.get("SVDQ_B200_ACT_LAYOUT")
    if _layout_env is not None and _layout_env[0] == raw:
        return _layout_env[1]
    v = (raw or "native").lower()
    if v not in ("native", "reference"):
        raise ValueError(f"SVDQ_B200_ACT_LAYOUT must be 'native' or 'reference', got {v!r}")
    _layout_env = (raw, _lib.LAYOUT_REFERENCE if v == "reference" else _lib.LAYOUT_NATIVE)
    return _layout_env[1]


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    """Raw cudaStream_t of torch's current stream on ``device`` (the entry points launch on it)."""
    idx = device.index
    if idx is None:
        idx = torch._C._cuda_getDevice()
    return torch._C._cuda_getCurrentRawStream(idx)


_NULL_CTX = contextlib.nullcontext()


def on_device(device: torch.device):
    """Context that makes ``device`` the current CUDA device; free when it already is (the entry points act on the
    current device, and switching through ``torch.cuda.device`` costs more than a launch)."""
    idx = device.index
    if idx is None or idx == torch._C._cuda_getDevice():
        return _NULL_CTX
    return torch.cuda.device(idx)


# The 16-bit floating-point types of the path (the reference's GEMMConfig_W4A4_BF16 / _FP16) and their C-ABI codes.
HALF_DTYPES = (torch.bfloat16, torch.float16)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 0
    if dtype == torch.float16:
        return 1
    raise ValueError(f"dtype {dtype}: the W4A4 path computes with bf16 or fp16 tensors")


def require_same_half_dtype(**tensors) -> torch.dtype | None:
    """All given (non-None) tensors share one of the two 16-bit types; returns it (None when there is no tensor)."""
    found = None
    for name, t in tensors.items():
        if t is None:
            continue
        if t.dtype not in HALF_DTYPES:
            raise ValueError(f"{name} has dtype {t.dtype}, expected one of {HALF_DTYPES}")
        if found is not None and t.dtype != found:
            raise ValueError(f"{name} has dtype {t.dtype} but other tensors of the call are {found}")
        found = t.dtype
    return found


def require_cuda_contiguous(name: str, t: torch.Tensor | None, dtypes=None) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
