"""Small host-side helpers (mirrors of nunchaku/utils.py:77-93 where they exist)."""
from __future__ import annotations

import os

import torch

from . import _lib


def ceil_divide(x: int, divisor: int) -> int:
    """nunchaku/utils.py:77-93."""
    return (x + divisor - 1) // divisor


def default_act_layout() -> int:
    """Memory order of the activation-side tensors handed from the quantiser to the GEMM.

    ``native`` (default) is what the sm_100a GEMM streams with TMA; ``reference`` is the
    reference's mma.sync fragment order (set ``SVDQ_B200_ACT_LAYOUT=reference``), which the
    GEMM converts back before use.
    """
    v = os.environ.get("SVDQ_B200_ACT_LAYOUT", "native").lower()
    if v not in ("native", "reference"):
        raise ValueError(f"SVDQ_B200_ACT_LAYOUT must be 'native' or 'reference', got {v!r}")
    return _lib.LAYOUT_REFERENCE if v == "reference" else _lib.LAYOUT_NATIVE


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda_contiguous(name: str, t: torch.Tensor | None, dtypes=None) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
