"""Fused call patterns built from the two W4A4 ops (mirror of ``nunchaku/ops/fused.py``)."""
from __future__ import annotations

import torch

from ..utils import ceil_divide
from .gemm import svdq_gemm_w4a4_cuda


def fused_gelu_mlp(x: torch.Tensor, fc1, fc2, pad_size: int = 256) -> torch.Tensor:
    """fc1 -> GELU -> fc2 with fc1's output kept 4-bit (``nunchaku/ops/fused.py:10-47``):
    fc1's GEMM epilogue applies GELU, the LoRA-down projection and the quantisation of
    fc2's input, so only codes, scales and the rank-R activations reach HBM."""
    batch_size, seq_len, channels = x.shape
    x = x.view(batch_size * seq_len, channels)
    quantized_x, ascales, lora_act = fc1.quantize(x)
    batch_size_pad = ceil_divide(batch_size * seq_len, pad_size) * pad_size
    dev = x.device
    qout_act = torch.empty(batch_size_pad, fc1.out_features // 2, dtype=torch.uint8, device=dev)
    if fc2.precision == "nvfp4":
        qout_ascales = torch.empty(fc1.out_features // 16, batch_size_pad, dtype=torch.float8_e4m3fn, device=dev)
    else:
        qout_ascales = torch.empty(fc1.out_features // 64, batch_size_pad, dtype=x.dtype, device=dev)
    qout_lora_act = torch.empty(batch_size_pad, fc2.proj_down.shape[1], dtype=torch.float32, device=dev)
    svdq_gemm_w4a4_cuda(
        act=quantized_x, wgt=fc1.qweight, qout=qout_act, ascales=ascales, wscales=fc1.wscales,
        oscales=qout_ascales, lora_act_in=lora_act, lora_up=fc1.proj_up, lora_down=fc2.proj_down,
        lora_act_out=qout_lora_act, bias=fc1.bias, smooth_factor=fc2.smooth_factor,
        fp4=fc1.precision == "nvfp4", alpha=fc1.wtscale, wcscales=fc1.wcscales,
        next_fp4=fc2.precision == "nvfp4",
    )
    output = torch.empty(batch_size * seq_len, fc2.out_features, dtype=x.dtype, device=dev)
    output = fc2.forward_quant(qout_act, qout_ascales, qout_lora_act, output=output)
    return output.view(batch_size, seq_len, -1)
