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


def qk_norm_rope(qkv: torch.Tensor, weight_q: torch.Tensor, weight_k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 heads: int, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm of q and k per 128-wide head and rotary embedding, in place on the output of a fused QKV projection
    (what ``fused_qkv_norm_rottary``, ``nunchaku/ops/fused.py:50-110``, gets from the GEMM epilogue).

    qkv: bf16 [B, S, 3*heads*128] (or [B*S, ...] with ``cos.shape[0]`` dividing the rows); cos, sin: fp32 [S, 64].
    """
    import ctypes

    from .. import _lib
    from ..utils import ptr, require_cuda_contiguous, stream_ptr

    require_cuda_contiguous("qkv", qkv, (torch.bfloat16,))
    require_cuda_contiguous("weight_q", weight_q, (torch.bfloat16,))
    require_cuda_contiguous("weight_k", weight_k, (torch.bfloat16,))
    require_cuda_contiguous("cos", cos, (torch.float32,))
    require_cuda_contiguous("sin", sin, (torch.float32,))
    if qkv.shape[-1] != 3 * heads * 128 or cos.shape != sin.shape or cos.shape[-1] != 64:
        raise ValueError("qk_norm_rope: qkv must be [..., 3*heads*128] and cos/sin [seq_len, 64]")
    rows = qkv.numel() // qkv.shape[-1]
    args = _lib.NormRopeArgs(qkv=ptr(qkv), weight_q=ptr(weight_q), weight_k=ptr(weight_k), cos=ptr(cos), sin=ptr(sin),
                             rows=rows, seq_len=cos.shape[0], heads=heads, eps=eps)
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().svdq_qk_norm_rope(ctypes.byref(args), stream_ptr(qkv.device)))
    return qkv


def layernorm_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``layer_norm(x) * (1 + scale) + shift`` (no affine) for x bf16 [B, S, C] and per-batch scale / shift bf16 [B, C]
    (views into a wider modulation tensor are fine as long as rows are contiguous)."""
    import ctypes

    from .. import _lib
    from ..utils import ptr, require_cuda_contiguous, stream_ptr

    require_cuda_contiguous("x", x, (torch.bfloat16,))
    B, S, C = x.shape
    if scale.shape != (B, C) or shift.shape != (B, C) or scale.stride(1) != 1 or shift.stride(1) != 1:
        raise ValueError("layernorm_modulate: scale / shift must be [B, C] with unit column stride")
    if scale.stride(0) != shift.stride(0) or scale.dtype != torch.bfloat16 or shift.dtype != torch.bfloat16:
        raise ValueError("layernorm_modulate: scale and shift must be bf16 views with the same row stride")
    out = torch.empty_like(x)
    args = _lib.LnModulateArgs(x=ptr(x), scale=scale.data_ptr(), shift=shift.data_ptr(), out=ptr(out), rows=B * S,
                               rows_per_batch=S, mod_stride=scale.stride(0) if B > 1 else max(scale.stride(0), C), cols=C, eps=eps)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().svdq_layernorm_modulate(ctypes.byref(args), stream_ptr(x.device)))
    return out


def litela_attention(qkv: torch.Tensor, heads: int, eps: float = 1e-6, return_vk: bool = False):
    """ReLU linear attention of SANA on the bf16 output of the fused QKV projection (what ``EpilogueLiteLA`` in the QKV
    GEMM plus ``linearattn_vk_mul_q`` compute for ``SanaLinearAttention::forward``, ``src/SanaModel.cpp:25-106``).

    qkv: bf16 [B, S, 3*heads*32], columns [Q of all heads | (K_h, V_h) 64 per head].  Returns bf16 [B, S, heads*32]
    (and the fp32 ``vk`` [B, heads, 33, 32] when asked)."""
    import ctypes

    from .. import _lib
    from ..utils import ptr, require_cuda_contiguous, stream_ptr

    require_cuda_contiguous("qkv", qkv, (torch.bfloat16,))
    if qkv.dim() != 3 or qkv.shape[-1] != 3 * heads * 32:
        raise ValueError("litela_attention: qkv must be [B, S, 3*heads*32]")
    B, S, _ = qkv.shape
    out = torch.empty(B, S, heads * 32, dtype=torch.bfloat16, device=qkv.device)
    vk = torch.empty(B, heads, 33, 32, dtype=torch.float32, device=qkv.device) if return_vk else None
    args = _lib.LiteLAArgs(qkv=ptr(qkv), out=ptr(out), vk=ptr(vk) if vk is not None else None, batches=B, tokens=S,
                           heads=heads, eps=eps)
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().svdq_litela(ctypes.byref(args), stream_ptr(qkv.device)))
    return (out, vk) if return_vk else out
