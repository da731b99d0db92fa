"""Softmax attention for 128-wide heads on the tcgen05 kernel of ``csrc/attention.cu``.

Mirrors ``nunchaku::ops::attention_fp16`` (nunchaku/csrc/ops.h:112-118, kernel src/kernels/zgemm/attention.cu:10-96; called
from nunchaku/models/attention_processors/flux.py:160-185).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..utils import HALF_DTYPES, dtype_code, on_device, stream_ptr

HEAD_DIM = 128


def _strides(name: str, t: torch.Tensor) -> tuple[int, int, int]:
    if t.dim() != 4 or t.shape[3] != HEAD_DIM or t.stride(3) != 1:
        raise ValueError(f"{name} must be [batch, heads, tokens, {HEAD_DIM}] (any strides, the last dimension contiguous)")
    s = [t.stride(0), t.stride(1), t.stride(2)]
    if t.shape[0] == 1:
        s[0] = 0
    if any(x % 8 for x in s) or t.data_ptr() % 16:
        raise ValueError(f"{name}: strides must be multiples of 8 elements and the data 16-byte aligned")
    return tuple(s)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None,
              scale: float | None = None) -> torch.Tensor:
    """``softmax(scale * q k^T) v`` per (batch, head).

    q: [B, H, Tq, 128]; k, v: [B, H, Tkv, 128], bf16 or fp16, as views with any (batch, head, token) strides: the reference's
    packed head-major tensors and token-major ``x.view(B, T, H, 128).transpose(1, 2)`` views are both taken as they are.
    out: [B, Tq, H*128] (default: a new tensor) or a [B, H, Tq, 128] view of one.  scale defaults to 128 ** -0.5."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda or t.dtype not in HALF_DTYPES or t.dtype != q.dtype:
            raise ValueError(f"{n} must be a CUDA bf16 / fp16 tensor of q's dtype")
    B, H, Tq, _ = q.shape
    if k.shape != v.shape or k.shape[0] != B or k.shape[1] != H:
        raise ValueError("k and v must be [batch, heads, tokens_kv, 128] with q's batch and heads")
    ret = out
    if out is None:
        ret = out = torch.empty(B, Tq, H * HEAD_DIM, dtype=q.dtype, device=q.device)
    if out.dim() == 3:
        if out.shape != (B, Tq, H * HEAD_DIM) or out.stride(2) != 1:
            raise ValueError("out must be [batch, tokens_q, heads*128] with unit channel stride")
        out = out.unflatten(2, (H, HEAD_DIM)).transpose(1, 2)
    if out.shape != q.shape or out.dtype != q.dtype or not out.is_cuda:
        raise ValueError("out must match q's shape (as [B, H, Tq, 128]) and dtype")
    args = _lib.AttentionArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                              q_stride=(ctypes.c_int64 * 3)(*_strides("q", q)), k_stride=(ctypes.c_int64 * 3)(*_strides("k", k)),
                              v_stride=(ctypes.c_int64 * 3)(*_strides("v", v)), o_stride=(ctypes.c_int64 * 3)(*_strides("out", out)),
                              batch=B, heads=H, q_len=Tq, kv_len=k.shape[2], head_dim=HEAD_DIM,
                              scale=float(HEAD_DIM ** -0.5 if scale is None else scale), dtype=dtype_code(q.dtype))
    with on_device(q.device):
        _lib.check(_lib.load().svdq_attention(ctypes.byref(args), stream_ptr(q.device)))
    return ret


def attention_fp16(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, scale: float) -> None:
    """The reference's call (nunchaku/csrc/ops.h:112-118): q, k, v packed [B, H, T, 128], o [B, Tq, H*128], written in place.
    The reference takes fp16 inputs with a bf16 or fp16 output; here all four share one 16-bit type."""
    attention(q, k, v, out=o, scale=scale)
