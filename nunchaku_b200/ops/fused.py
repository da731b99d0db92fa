"""Fused call patterns built from the two W4A4 ops (mirror of ``nunchaku/ops/fused.py``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..utils import HALF_DTYPES, ceil_divide, dtype_code, on_device, ptr, require_cuda_contiguous, stream_ptr
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


def fused_qkv_norm_rottary(x: torch.Tensor, proj, norm_q, norm_k, rotary_emb: torch.Tensor,
                           output: torch.Tensor | tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                           attn_tokens: int = 0):
    """Fused QKV projection + RMSNorm of q / k per head + rotary embedding (``nunchaku/ops/fused.py:50-110``, the
    name is the reference's).  ``norm_q`` / ``norm_k`` are RMSNorm modules (their ``weight`` [128] is used),
    ``rotary_emb`` is the packed fp32 tensor of ``pack_rotemb`` with ``shape[0] * shape[1]`` equal to the padded row
    count.  ``output`` is a [rows, 3*dim] tensor (default: allocated), or a tuple ``(out_q, out_k, out_v)`` of
    head-major [B, heads, tokens_pad, 128] tensors."""
    batch_size, seq_len, channels = x.shape
    x = x.view(batch_size * seq_len, channels)
    quantized_x, ascales, lora_act = proj.quantize(x)
    if output is None:
        output = torch.empty(quantized_x.shape[0], proj.out_features, dtype=x.dtype, device=x.device)
    common = dict(act=quantized_x, wgt=proj.qweight, ascales=ascales, wscales=proj.wscales, lora_act_in=lora_act,
                  lora_up=proj.proj_up, bias=proj.bias, fp4=proj.precision == "nvfp4", alpha=proj.wtscale,
                  wcscales=proj.wcscales, norm_q=norm_q.weight, norm_k=norm_k.weight, rotary_emb=rotary_emb)
    if isinstance(output, tuple):
        if len(output) != 3:
            raise ValueError("output must be (out_q, out_k, out_v)")
        svdq_gemm_w4a4_cuda(out_q=output[0], out_k=output[1], out_v=output[2], attn_tokens=attn_tokens, **common)
        return output
    svdq_gemm_w4a4_cuda(out=output, **common)
    return output.view(batch_size, seq_len, -1)


def qkv_proj_norm_rope(x: torch.Tensor, proj, weight_q: torch.Tensor, weight_k: torch.Tensor, cos: torch.Tensor,
                       sin: torch.Tensor, heads: int, eps: float = 1e-6,
                       out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None, token_offset: int = 0):
    """Fused QKV projection of ``x`` [B, S, C] through the W4A4 layer ``proj`` with RMSNorm of q / k per 128-wide head and the
    rotary embedding from plain tables (cos, sin fp32 [S, 64]): one quantiser launch and one GEMM whose epilogue does the
    rest (a second row-wise kernel only for shapes the fused epilogue is not built for).  Returns the [B, S, 3*C'] tensor,
    or None when ``out = (q, k, v)`` (token-major [B, S_total, heads*128] buffers filled from ``token_offset`` on)."""
    B, S, C = x.shape
    quantized_x, ascales, lora_act = proj.quantize(x.reshape(B * S, C))
    tile = None if out is not None else torch.empty(B * S, proj.out_features, dtype=x.dtype, device=x.device)
    svdq_gemm_w4a4_cuda(act=quantized_x, wgt=proj.qweight, out=tile, ascales=ascales, wscales=proj.wscales, lora_act_in=lora_act,
                        lora_up=proj.proj_up, bias=proj.bias, fp4=proj.precision == "nvfp4", alpha=proj.wtscale,
                        wcscales=proj.wcscales, norm_q=weight_q, norm_k=weight_k, rope_cos=cos, rope_sin=sin, rope_heads=heads,
                        rope_eps=eps, rope_out=out, rope_token_offset=token_offset)
    return None if tile is None else tile.view(B, S, -1)


def unpack_rotemb(rotary_emb: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The reference's fragment-packed rotary tensor (``pack_rotemb``, nunchaku/models/embeddings.py:88-120) as plain
    (cos, sin) tables fp32 [rows, 64]: for row m = 16 mb + 8 h + g and pair p = 4 j + t, {sin, cos} sit at
    ((((mb*16 + j)*8 + g)*4 + t)*2 + h)*2.  Cached on the tensor (per version)."""
    cached = rotary_emb.__dict__.get("_svdq_b200_tables")
    if cached is not None and cached[0] == rotary_emb._version:
        return cached[1], cached[2]
    rows = rotary_emb.shape[0] * rotary_emb.shape[1]
    t = rotary_emb.reshape(rows // 16, 16, 8, 4, 2, 2).permute(0, 4, 2, 1, 3, 5).reshape(rows, 64, 2)
    sin, cos = t[..., 0].contiguous(), t[..., 1].contiguous()
    rotary_emb.__dict__["_svdq_b200_tables"] = (rotary_emb._version, cos, sin)
    return cos, sin


def _norm_rope_packed(qkv, norm_q, norm_k, rotary_emb, out_q, out_k, out_v, attn_tokens: int) -> None:
    """The RMSNorm + RoPE (+ head-major split) step of the QKV epilogue on the projection's bf16 tile ``qkv`` [rows, 3*dim],
    with the reference's packed rotary tensor [B_r, M_r, 128] (B_r * M_r rows; the table repeats over ``qkv``'s rows)."""
    require_cuda_contiguous("norm_q", norm_q, (qkv.dtype,))
    require_cuda_contiguous("norm_k", norm_k, (qkv.dtype,))
    require_cuda_contiguous("rotary_emb", rotary_emb, (torch.float32,))
    if rotary_emb.dim() != 3 or rotary_emb.shape[2] != 128:
        raise ValueError("rotary_emb must be the packed fp32 tensor [B, M, 128] (gemm_w4a4_launch_impl.cuh:351-354)")
    rows = qkv.numel() // qkv.shape[-1]
    table_rows = rotary_emb.shape[0] * rotary_emb.shape[1]
    dim = qkv.shape[-1] // 3
    if dim % 128 or rows % table_rows:
        raise ValueError("the QKV width must be 3 * heads * 128 and the row count a multiple of the rotary table's rows")
    heads = dim // 128
    args = _lib.NormRopeArgs(qkv=ptr(qkv), weight_q=ptr(norm_q), weight_k=ptr(norm_k), cos=None, sin=None, rows=rows,
                             seq_len=table_rows, heads=heads, eps=1e-6, rotary_packed=ptr(rotary_emb), dtype=dtype_code(qkv.dtype))
    if out_q is not None:
        for n, t in (("out_q", out_q), ("out_k", out_k), ("out_v", out_v)):
            if t is None:
                raise ValueError("out_q, out_k and out_v go together")
            require_cuda_contiguous(n, t, (qkv.dtype,))
            if t.dim() != 4 or t.shape[1] != heads or t.shape[3] != 128 or t.shape[0] * table_rows != rows or t.shape[2] < table_rows:
                raise ValueError(f"{n} must be [rows / table rows, heads, tokens_pad >= table rows, 128]")
        args.out_q, args.out_k, args.out_v = ptr(out_q), ptr(out_k), ptr(out_v)
        args.tokens_pad = out_q.shape[2]
        args.attn_tokens = attn_tokens
    _lib.check(_lib.load().svdq_qk_norm_rope(ctypes.byref(args), stream_ptr(qkv.device)))


def _litela_epilogue(qkv: torch.Tensor, out_vk: torch.Tensor, out_linearattn: torch.Tensor) -> None:
    """What ``EpilogueLiteLA`` leaves behind (gemm_w4a4_launch_impl.cuh:311-345): ``out_vk`` [B, heads, 33, 32] fp32 and
    relu(Q) in ``out_linearattn`` [B, tokens, N/3], from the projection's 16-bit tile ``qkv`` [B*tokens, N] (same dtype)."""
    require_cuda_contiguous("out_vk", out_vk, (torch.float32,))
    require_cuda_contiguous("out_linearattn", out_linearattn, (qkv.dtype,))
    if out_vk.dim() != 4 or out_vk.shape[2:] != (33, 32) or out_linearattn.dim() != 3:
        raise ValueError("out_vk must be [B, heads, 33, 32] and out_linearattn [B, tokens, N/3]")
    B, heads = out_vk.shape[0], out_vk.shape[1]
    tokens = out_linearattn.shape[1]
    if heads * 96 != qkv.shape[-1] or out_linearattn.shape != (B, tokens, heads * 32) or qkv.numel() != B * tokens * heads * 96:
        raise ValueError("linear attention: N must be 3 * heads * 32 and the rows B * tokens")
    args = _lib.LiteLAArgs(qkv=ptr(qkv), out=ptr(out_linearattn), vk=ptr(out_vk), batches=B, tokens=tokens, heads=heads,
                           eps=1e-6, mode=1, dtype=dtype_code(qkv.dtype))
    _lib.check(_lib.load().svdq_litela(ctypes.byref(args), stream_ptr(qkv.device)))


def linearattn_vk_mul_q(q: torch.Tensor, vk: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """In place on ``q`` [B, tokens, heads*32] (relu(Q), bf16 or fp16): ``o = q @ vk^T`` per head, ``q <- o[:32] / (o[32] + eps)``
    (``linearattn_vk_mul_q``, gemm_w4a4_launch_impl.cuh:426-448; ``vk_mul_q_kernel``, epilogues.cuh:704-759)."""
    require_cuda_contiguous("q", q, HALF_DTYPES)
    require_cuda_contiguous("vk", vk, (torch.float32,))
    B, tokens, D = q.shape
    if vk.shape != (B, D // 32, 33, 32):
        raise ValueError("vk must be [B, heads, 33, 32]")
    args = _lib.LiteLAArgs(qkv=None, out=ptr(q), vk=ptr(vk), batches=B, tokens=tokens, heads=D // 32, eps=eps, mode=2,
                           dtype=dtype_code(q.dtype))
    with on_device(q.device):
        _lib.check(_lib.load().svdq_litela(ctypes.byref(args), stream_ptr(q.device)))
    return q


def qk_norm_rope(qkv: torch.Tensor, weight_q: torch.Tensor, weight_k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 heads: int, eps: float = 1e-6, out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                 token_offset: int = 0) -> torch.Tensor:
    """RMSNorm of q and k per 128-wide head and rotary embedding, in place on the output of a fused QKV projection
    (what ``fused_qkv_norm_rottary``, ``nunchaku/ops/fused.py:50-110``, gets from the GEMM epilogue).

    qkv: bf16 or fp16 [B, S, 3*heads*128] (or [B*S, ...] with ``cos.shape[0]`` dividing the rows); cos, sin: fp32 [S, 64].
    With ``out = (q, k, v)``, three [B, S_total, heads*128] buffers of qkv's dtype, the three thirds are written there instead
    (token-major, rows ``token_offset .. token_offset + S``): the two streams of a joint block fill one set of buffers
    that attention reads without any concatenation.
    """
    require_cuda_contiguous("qkv", qkv, HALF_DTYPES)
    require_cuda_contiguous("weight_q", weight_q, (qkv.dtype,))
    require_cuda_contiguous("weight_k", weight_k, (qkv.dtype,))
    require_cuda_contiguous("cos", cos, (torch.float32,))
    require_cuda_contiguous("sin", sin, (torch.float32,))
    if qkv.shape[-1] != 3 * heads * 128 or cos.shape != sin.shape or cos.shape[-1] != 64:
        raise ValueError("qk_norm_rope: qkv must be [..., 3*heads*128] and cos/sin [seq_len, 64]")
    rows = qkv.numel() // qkv.shape[-1]
    args = _lib.NormRopeArgs(qkv=ptr(qkv), weight_q=ptr(weight_q), weight_k=ptr(weight_k), cos=ptr(cos), sin=ptr(sin),
                             rows=rows, seq_len=cos.shape[0], heads=heads, eps=eps, dtype=dtype_code(qkv.dtype))
    if out is not None:
        for t in out:
            require_cuda_contiguous("out", t, (qkv.dtype,))
            if t.dim() != 3 or t.shape[2] != heads * 128 or t.shape[0] * cos.shape[0] != rows:
                raise ValueError("qk_norm_rope: out tensors must be [rows / S, S_total, heads*128]")
        args.out_q, args.out_k, args.out_v = ptr(out[0]), ptr(out[1]), ptr(out[2])
        args.tokens_pad, args.token_offset, args.token_major = out[0].shape[1], token_offset, 1
    with on_device(qkv.device):
        _lib.check(_lib.load().svdq_qk_norm_rope(ctypes.byref(args), stream_ptr(qkv.device)))
    return qkv


def layernorm_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``layer_norm(x) * (1 + scale) + shift`` (no affine) for x bf16 or fp16 [B, S, C] and per-batch scale / shift [B, C] of
    the same dtype (views into a wider modulation tensor are fine as long as rows are contiguous)."""
    require_cuda_contiguous("x", x, HALF_DTYPES)
    B, S, C = x.shape
    if scale.shape != (B, C) or shift.shape != (B, C) or scale.stride(1) != 1 or shift.stride(1) != 1:
        raise ValueError("layernorm_modulate: scale / shift must be [B, C] with unit column stride")
    if scale.stride(0) != shift.stride(0) or scale.dtype != x.dtype or shift.dtype != x.dtype:
        raise ValueError("layernorm_modulate: scale and shift must be views of x's dtype with the same row stride")
    out = torch.empty_like(x)
    args = _lib.LnModulateArgs(x=ptr(x), scale=scale.data_ptr(), shift=shift.data_ptr(), out=ptr(out), rows=B * S,
                               rows_per_batch=S, mod_stride=scale.stride(0) if B > 1 else max(scale.stride(0), C), cols=C, eps=eps,
                               dtype=dtype_code(x.dtype))
    with on_device(x.device):
        _lib.check(_lib.load().svdq_layernorm_modulate(ctypes.byref(args), stream_ptr(x.device)))
    return out


def gate_residual(x: torch.Tensor, gate: torch.Tensor | None, y: torch.Tensor, z: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """``x + gate[:, None, :] * (y (+ z))`` for bf16 or fp16 x, y, z [B, S, C] and a per-batch gate [B, C] of the same dtype (a view
    with unit column stride is fine; None = 1): the gated residual after a projection, in one pass.  ``out`` defaults to a new tensor and may
    be ``x``."""
    require_cuda_contiguous("x", x, HALF_DTYPES)
    require_cuda_contiguous("y", y, (x.dtype,))
    require_cuda_contiguous("z", z, (x.dtype,))
    B, S, C = x.shape
    if y.shape != x.shape or (z is not None and z.shape != x.shape) or C % 8:
        raise ValueError("gate_residual: x, y, z must be [B, S, C] with C a multiple of 8")
    stride = 0
    if gate is not None:
        if gate.shape != (B, C) or gate.stride(1) != 1 or gate.dtype != x.dtype or not gate.is_cuda:
            raise ValueError("gate_residual: gate must be a [B, C] view of x's dtype with unit column stride")
        stride = gate.stride(0) if B > 1 else max(gate.stride(0), C)
    if out is None:
        out = torch.empty_like(x)
    args = _lib.GateResidualArgs(x=ptr(x), gate=None if gate is None else gate.data_ptr(), y=ptr(y), z=ptr(z), out=ptr(out),
                                 rows=B * S, rows_per_batch=S, gate_stride=stride, cols=C, dtype=dtype_code(x.dtype))
    with on_device(x.device):
        _lib.check(_lib.load().svdq_gate_residual(ctypes.byref(args), stream_ptr(x.device)))
    return out


def litela_attention(qkv: torch.Tensor, heads: int, eps: float = 1e-6, return_vk: bool = False):
    """ReLU linear attention of SANA on the bf16 output of the fused QKV projection (what ``EpilogueLiteLA`` in the QKV
    GEMM plus ``linearattn_vk_mul_q`` compute for ``SanaLinearAttention::forward``, ``src/SanaModel.cpp:25-106``).

    qkv: bf16 or fp16 [B, S, 3*heads*32], columns [Q of all heads | (K_h, V_h) 64 per head].  Returns [B, S, heads*32] of the
    same dtype (and the fp32 ``vk`` [B, heads, 33, 32] when asked)."""
    require_cuda_contiguous("qkv", qkv, HALF_DTYPES)
    if qkv.dim() != 3 or qkv.shape[-1] != 3 * heads * 32:
        raise ValueError("litela_attention: qkv must be [B, S, 3*heads*32]")
    B, S, _ = qkv.shape
    out = torch.empty(B, S, heads * 32, dtype=qkv.dtype, device=qkv.device)
    vk = torch.empty(B, heads, 33, 32, dtype=torch.float32, device=qkv.device) if return_vk else None
    args = _lib.LiteLAArgs(qkv=ptr(qkv), out=ptr(out), vk=ptr(vk) if vk is not None else None, batches=B, tokens=S,
                           heads=heads, eps=eps, dtype=dtype_code(qkv.dtype))
    with on_device(qkv.device):
        _lib.check(_lib.load().svdq_litela(ctypes.byref(args), stream_ptr(qkv.device)))
    return (out, vk) if return_vk else out
