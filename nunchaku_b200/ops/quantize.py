"""Python wrapper of the activation quantiser; same signature and return value as
``nunchaku/ops/quantize.py:11-54`` (``svdq_quantize_w4a4_act_fuse_lora_cuda``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..utils import ceil_divide, default_act_layout, on_device, ptr, require_cuda_contiguous, stream_ptr, HALF_DTYPES, dtype_code, require_same_half_dtype


def svdq_quantize_w4a4_act_fuse_lora_cuda(
    input: torch.Tensor,
    output: torch.Tensor | None = None,
    oscales: torch.Tensor | None = None,
    lora_down: torch.Tensor | None = None,
    lora_act_out: torch.Tensor | None = None,
    smooth: torch.Tensor | None = None,
    fuse_glu: bool = False,
    fp4: bool = False,
    pad_size: int = 256,
    layout: int | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantise ``input`` [M, K] (bf16) to 4-bit codes + group scales and apply the LoRA
    down projection.

    ``lora_down`` ([K, R]) and ``smooth`` ([K]) are the packed module parameters
    ``SVDQW4A4Linear.proj_down`` / ``.smooth_factor``.  Returns ``(output, oscales,
    lora_act_out)`` with the reference's shapes: uint8 [M_pad, K/2]; float8_e4m3fn
    [K/16, M_pad] (NVFP4) or bf16 [K/64, M_pad] (INT4); fp32 [M_pad, R].  ``layout``
    selects their memory order (default: :func:`nunchaku_b200.utils.default_act_layout`).
    """
    if lora_down is None or smooth is None:
        raise ValueError("lora_down and smooth are required (the reference dereferences both)")
    require_cuda_contiguous("input", input, HALF_DTYPES)
    require_cuda_contiguous("lora_down", lora_down, HALF_DTYPES)
    require_cuda_contiguous("smooth", smooth, HALF_DTYPES)
    half = require_same_half_dtype(input=input, lora_down=lora_down, smooth=smooth)
    if input.dim() != 2:
        raise ValueError("input must be 2-D [M, K]")
    batch_size, channels = input.shape
    if fuse_glu:
        channels //= 2
    # an input narrower than the (128-padded) parameters is read as if padded with zero columns
    # (in_features vs in_features_pad, src/Linear.cpp:92,452)
    k_in = 0
    if smooth.numel() != channels and 0 < smooth.numel() - channels < 128:
        k_in, channels = channels, smooth.numel()
    rank = lora_down.shape[1]
    batch_size_pad = ceil_divide(batch_size, pad_size) * pad_size
    dev = input.device
    if output is None:
        output = torch.empty(batch_size_pad, channels // 2, dtype=torch.uint8, device=dev)
    if oscales is None:
        if fp4:
            if channels % 16 != 0:
                raise ValueError("channels must be a multiple of 16")
            oscales = torch.empty(channels // 16, batch_size_pad, dtype=torch.float8_e4m3fn, device=dev)
        else:
            if channels % 64 != 0:
                raise ValueError("channels must be a multiple of 64")
            oscales = torch.empty(channels // 64, batch_size_pad, dtype=input.dtype, device=dev)
    if lora_act_out is None:
        lora_act_out = torch.empty(batch_size_pad, rank, dtype=torch.float32, device=dev)
    require_cuda_contiguous("output", output, (torch.uint8, torch.int8))
    require_cuda_contiguous("oscales", oscales, (torch.float8_e4m3fn,) if fp4 else (half,))
    require_cuda_contiguous("lora_act_out", lora_act_out, (torch.float32,))
    if output.numel() != batch_size_pad * channels // 2 or lora_act_out.numel() != batch_size_pad * rank:
        raise ValueError("output / lora_act_out have the wrong number of elements")
    if oscales.numel() != batch_size_pad * channels // (16 if fp4 else 64):
        raise ValueError("oscales has the wrong number of elements")

    args = _lib.QuantizeArgs(
        input=ptr(input), codes=ptr(output), scales=ptr(oscales), lora_act=ptr(lora_act_out),
        smooth=ptr(smooth), lora_down=ptr(lora_down),
        M=batch_size, M_pad=batch_size_pad, K=channels, R=rank,
        fp4=int(fp4), fuse_glu=int(fuse_glu),
        layout=default_act_layout() if layout is None else layout, K_in=k_in, dtype=dtype_code(half),
    )
    with on_device(dev):
        _lib.check(_lib.load().svdq_quantize_w4a4_act_fuse_lora(ctypes.byref(args), stream_ptr(dev)))
    return output, oscales, lora_act_out


def svdq_quantize_w4a4_wgt(input: torch.Tensor, output: torch.Tensor | None = None,
                           oscales: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """INT4 weight quantiser: bf16 / fp16 ``input`` [N, K] -> (``qweight`` int8 [N, K/2], ``wscales`` [K/64, N] of the input's
    dtype), both in the packed layouts of ``SVDQW4A4Linear``'s parameters (``nunchaku::kernels::quantize_w4a4_wgt``,
    src/kernels/zgemm/zgemm.h:48: input, output, oscales in that order, written in place when given).  Arithmetic as the
    reference's kernel does it, in the 16-bit type: scale = max|w| / 7, code = sat_s4(rint(w * (7 / max|w|)))."""
    require_cuda_contiguous("input", input, HALF_DTYPES)
    if input.dim() != 2 or input.shape[0] % 128 or input.shape[1] % 64:
        raise ValueError("input must be [N, K] with N a multiple of 128 and K of 64")
    N, K = input.shape
    if output is None:
        output = torch.empty(N, K // 2, dtype=torch.int8, device=input.device)
    if oscales is None:
        oscales = torch.empty(K // 64, N, dtype=input.dtype, device=input.device)
    require_cuda_contiguous("output", output, (torch.int8, torch.uint8))
    require_cuda_contiguous("oscales", oscales, (input.dtype,))
    if output.numel() != N * K // 2 or oscales.numel() != N * K // 64:
        raise ValueError("output must hold N * K / 2 bytes and oscales N * K / 64 values")
    args = _lib.QuantizeWgtArgs(input=ptr(input), qweight=ptr(output), wscales=ptr(oscales), N=N, K=K, dtype=dtype_code(input.dtype))
    with on_device(input.device):
        _lib.check(_lib.load().svdq_quantize_w4a4_wgt(ctypes.byref(args), stream_ptr(input.device)))
    return output, oscales
