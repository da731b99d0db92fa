"""Python wrapper of the W4A4 GEMM; same signature as ``nunchaku/ops/gemm.py:12-159``
(``svdq_gemm_w4a4_cuda``).

Weights arrive in the reference's packed order (the checkpoint format).  The sm_100a
kernel streams K-major tiles with TMA, so each layer's weights are re-tiled once
(`svdq_w4a4_prepare_weights`).  The re-tiled copy hangs off the packed ``qweight`` tensor
itself (an attribute of the parameter object), so it lives and dies with the layer; it is
rebuilt when any of the packed tensors is replaced or modified in place.  A write through
``param.data`` does not bump the tensor's version counter: after such a write call
:func:`invalidate_prepared` (``SVDQW4A4Linear`` does it when a state dict is loaded).
"""
from __future__ import annotations

import ctypes
import math
import threading

import torch

from .. import _lib
from ..utils import default_act_layout, on_device, ptr, require_cuda_contiguous, stream_ptr, HALF_DTYPES, dtype_code, require_same_half_dtype

_ATTR = "_svdq_b200_prepared"
_lock = threading.Lock()   # guards creation / replacement of a layer's prepared weights (the C entry points are re-entrant)


class PreparedWeights:
    """Device buffers holding one layer's weights in the kernel's streaming order, plus the host-side state a call
    needs: a pre-filled argument struct and the scratch sizes already asked for."""

    def __init__(self, N: int, K: int, R: int, fp4: bool, device: torch.device):
        sizes = (ctypes.c_size_t * 5)()
        _lib.check(_lib.load().svdq_w4a4_prepared_bytes(N, K, R, int(fp4), sizes))
        self.N, self.K, self.R, self.fp4 = N, K, R, fp4
        self.device = device
        self.wgt = torch.empty(sizes[0], dtype=torch.uint8, device=device)
        self.wscales = torch.empty(sizes[1], dtype=torch.uint8, device=device)
        self.lora_up = torch.empty(max(sizes[2], 16), dtype=torch.uint8, device=device)
        self.col_scale = torch.empty(sizes[3], dtype=torch.uint8, device=device)
        self.col_bias = torch.empty(sizes[4], dtype=torch.uint8, device=device)
        self.workspace_bytes: dict[tuple, int] = {}
        self.key = None
        self.tls = threading.local()   # per-thread argument struct (two threads may run the same layer)

    def as_struct(self) -> _lib.PreparedWeights:
        return _lib.PreparedWeights(
            wgt=ptr(self.wgt), wscales=ptr(self.wscales), lora_up=ptr(self.lora_up) if self.R else None,
            col_scale=ptr(self.col_scale), col_bias=ptr(self.col_bias),
        )

    def args(self) -> _lib.GemmArgs:
        a = getattr(self.tls, "args", None)
        if a is None:
            a = _lib.GemmArgs(w=self.as_struct(), N=self.N, K=self.K, R=self.R, fp4=int(self.fp4))
            self.tls.args = a
            self.tls.ref = ctypes.byref(a)
        return a


def prepare_weights(
    wgt: torch.Tensor,
    wscales: torch.Tensor,
    lora_up: torch.Tensor | None,
    bias: torch.Tensor | None,
    wcscales: torch.Tensor | None,
    alpha: float,
    lora_scales: list[float] | None,
    fp4: bool,
) -> PreparedWeights:
    require_cuda_contiguous("wgt", wgt, (torch.int8, torch.uint8))
    require_cuda_contiguous("wscales", wscales, (torch.float8_e4m3fn,) if fp4 else HALF_DTYPES)
    require_cuda_contiguous("lora_up", lora_up)
    require_cuda_contiguous("bias", bias)
    require_cuda_contiguous("wcscales", wcscales)
    half = require_same_half_dtype(wscales=None if fp4 else wscales, lora_up=lora_up, bias=bias, wcscales=wcscales) or torch.bfloat16
    N, K = wgt.shape[0], wgt.shape[1] * 2
    R = 0 if lora_up is None else lora_up.shape[1]
    out = PreparedWeights(N, K, R, fp4, wgt.device)
    ls = None
    if lora_scales is not None and not all(s == 1.0 for s in lora_scales):
        ls = (ctypes.c_float * len(lora_scales))(*lora_scales)
    args = _lib.WeightsArgs(
        qweight=ptr(wgt), wscales=ptr(wscales), lora_up=ptr(lora_up), bias=ptr(bias), wcscales=ptr(wcscales),
        lora_scales=ls, alpha=float(alpha), N=N, K=K, R=R, fp4=int(fp4), dtype=dtype_code(half),
    )
    out.half_dtype = half
    st = out.as_struct()
    with on_device(wgt.device):
        _lib.check(_lib.load().svdq_w4a4_prepare_weights(ctypes.byref(args), ctypes.byref(st), stream_ptr(wgt.device)))
    return out


def _alpha_value(alpha) -> float:
    """``alpha`` is ``SVDQW4A4Linear.wtscale`` (a CUDA parameter) or a float.  The reference converts the tensor to
    a C++ float on every call (an implicit device sync, nunchaku/csrc/ops.h:33); here the value is read when the
    layer's weights are (re-)prepared, i.e. once per tensor object and version."""
    if alpha is None:
        return 1.0
    if isinstance(alpha, torch.Tensor):
        return float(alpha.detach().float().reshape(-1)[0].item())
    return float(alpha)


def _key(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4):
    """Identity (object ids, kept alive by the entry itself) and version of everything the prepared copy was built from."""
    ts = (wgt, wscales, lora_up, bias, wcscales, alpha if isinstance(alpha, torch.Tensor) else None)
    return (tuple(None if t is None else t._version for t in ts), None if isinstance(alpha, torch.Tensor) else alpha,
            None if lora_scales is None else tuple(lora_scales), bool(fp4))


def cached_prepared_weights(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4) -> PreparedWeights:
    hit = wgt.__dict__.get(_ATTR)
    key = _key(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4)
    if hit is not None:
        prepared, others = hit
        o = others
        if (prepared.key == key and o[0] is wscales and o[1] is lora_up and o[2] is bias and o[3] is wcscales
                and (o[4] is alpha or not isinstance(alpha, torch.Tensor))):
            return prepared
    with _lock:
        prepared = prepare_weights(wgt, wscales, lora_up, bias, wcscales, _alpha_value(alpha), lora_scales, fp4)
        prepared.key = key
        # the entry keeps the companion tensors alive, so `is` comparisons cannot be fooled by a recycled address;
        # the entry itself is owned by `wgt` and goes away with it (no reference from `others` back to `wgt`)
        setattr(wgt, _ATTR, (prepared, (wscales, lora_up, bias, wcscales, alpha if isinstance(alpha, torch.Tensor) else None)))
    return prepared


def invalidate_prepared(*tensors: torch.Tensor | None) -> None:
    """Drop the re-tiled copy that hangs off each given packed ``qweight``: needed after a write that does not go
    through the tensor's version counter (``param.data.copy_()``, ``param.data = ...``, a raw pointer)."""
    for t in tensors:
        if t is not None:
            t.__dict__.pop(_ATTR, None)


def clear_prepared_cache(module: torch.nn.Module | None = None) -> None:
    """Drop the prepared weights of every ``qweight`` below ``module`` (with no argument there is nothing global to
    clear: the copies are owned by the parameters)."""
    if module is None:
        return
    for name, p in module.named_parameters():
        if name.endswith("qweight"):
            invalidate_prepared(p)


def relayout_act(codes, scales, lora_act, K: int, fp4: bool, from_layout: int, to_layout: int):
    """Convert (codes, scales, lora_act) between the reference and the native memory order."""
    co = torch.empty_like(codes)
    so = torch.empty_like(scales)
    lo = torch.empty_like(lora_act) if lora_act is not None else None
    args = _lib.RelayoutArgs(
        codes_in=ptr(codes), codes_out=ptr(co), scales_in=ptr(scales), scales_out=ptr(so),
        lora_in=ptr(lora_act), lora_out=ptr(lo),
        M_pad=codes.shape[0], K=K, R=0 if lora_act is None else lora_act.shape[1], fp4=int(fp4),
        from_layout=from_layout, to_layout=to_layout,
    )
    with on_device(codes.device):
        _lib.check(_lib.load().svdq_w4a4_relayout_act(ctypes.byref(args), stream_ptr(codes.device)))
    return co, so, lo


def _gemm_rope_tables(a, lib, prepared, dev, out, norm_q, norm_k, cos, sin, heads, eps, rope_out, token_offset, M_pad, N) -> bool:
    """The QKV projection with RMSNorm + rotary embedding from plain (cos, sin) tables.  Returns True when done: either
    inside the GEMM's epilogue, or (shapes the fused epilogue is not built for) by the GEMM into a tile followed by the
    row-wise kernel."""
    from .fused import qk_norm_rope

    if norm_q is None or norm_k is None or sin is None or heads <= 0:
        raise ValueError("rope_cos needs rope_sin, norm_q, norm_k and rope_heads")
    require_cuda_contiguous("rope_cos", cos, (torch.float32,))
    require_cuda_contiguous("rope_sin", sin, (torch.float32,))
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != 64 or N != 3 * heads * 128:
        raise ValueError("rope tables must be fp32 [S, 64] and N = 3 * heads * 128")
    S = cos.shape[0]
    rows = a.M
    if rope_out is not None:
        for t in rope_out:
            require_cuda_contiguous("rope_out", t, HALF_DTYPES)
            if t.dim() != 3 or t.shape[2] != heads * 128 or t.shape[0] * S != rows or t.shape[1] < token_offset + S:
                raise ValueError("rope_out tensors must be [rows / S, S_total >= token_offset + S, heads*128]")
    elif out is None:
        raise ValueError("rope_cos needs `out` or `rope_out`")
    a.rope_norm_q, a.rope_norm_k = norm_q.data_ptr(), norm_k.data_ptr()
    a.rope_cos, a.rope_sin = cos.data_ptr(), sin.data_ptr()
    a.rope_eps, a.rope_seq_len, a.rope_heads = eps, S, heads
    a.rope_attn_tokens = 0
    if rope_out is not None:
        a.rope_out_q, a.rope_out_k, a.rope_out_v = (t.data_ptr() for t in rope_out)
        a.rope_tokens_pad, a.rope_token_offset = rope_out[0].shape[1], token_offset
    else:
        a.rope_out_q = a.rope_out_k = a.rope_out_v = None
        a.rope_tokens_pad = a.rope_token_offset = 0
    with on_device(dev):
        try:
            _lib.check(lib.svdq_gemm_w4a4(prepared.tls.ref, stream_ptr(dev)))
            return True
        except NotImplementedError:
            pass
        # not a shape of the fused epilogue: plain projection, then the row-wise kernel on its tile
        a.rope_cos = None
        tile = out
        if tile is None:
            tile = torch.empty(rows, N, dtype=rope_out[0].dtype, device=dev)
            a.out = tile.data_ptr()
        _lib.check(lib.svdq_gemm_w4a4(prepared.tls.ref, stream_ptr(dev)))
        qk_norm_rope(tile, norm_q, norm_k, cos, sin, heads, eps=eps, out=rope_out, token_offset=token_offset)
    return True


def svdq_gemm_w4a4_cuda(
    act: torch.Tensor,
    wgt: torch.Tensor,
    out: torch.Tensor | None = None,
    qout: torch.Tensor | None = None,
    ascales: torch.Tensor | None = None,
    wscales: torch.Tensor | None = None,
    oscales: torch.Tensor | None = None,
    poolout: torch.Tensor | None = None,
    lora_act_in: torch.Tensor | None = None,
    lora_up: torch.Tensor | None = None,
    lora_down: torch.Tensor | None = None,
    lora_act_out: torch.Tensor | None = None,
    norm_q: torch.Tensor | None = None,
    norm_k: torch.Tensor | None = None,
    rotary_emb: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    smooth_factor: torch.Tensor | None = None,
    out_vk: torch.Tensor | None = None,
    out_linearattn: torch.Tensor | None = None,
    act_unsigned: bool = False,
    lora_scales: list[float] | None = None,
    fuse_silu: bool = False,
    fp4: bool = False,
    alpha: float | torch.Tensor | None = 1.0,
    wcscales: torch.Tensor | None = None,
    out_q: torch.Tensor | None = None,
    out_k: torch.Tensor | None = None,
    out_v: torch.Tensor | None = None,
    attn_tokens: int = 0,
    act_layout: int | None = None,
    out_layout: int | None = None,
    next_fp4: bool | None = None,
    rope_cos: torch.Tensor | None = None,
    rope_sin: torch.Tensor | None = None,
    rope_heads: int = 0,
    rope_eps: float = 1e-6,
    rope_out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
    rope_token_offset: int = 0,
) -> None:
    """W4A4 GEMM with the fused SVDQuant epilogue; results are written in place.

    Argument meaning follows the reference (``GEMM_W4A4_Launch::gemm_w4a4``,
    gemm_w4a4_launch_impl.cuh:7-424), including which arguments select which epilogue:

    * ``qout`` + ``oscales`` (+ ``lora_down``, ``lora_act_out``, ``smooth_factor``): GELU and the next layer's
      LoRA-down + requantisation (launch_impl.cuh:282-309); ``out`` may be given as well;
    * ``out_linearattn`` + ``out_vk``: SANA's ReLU linear attention (launch_impl.cuh:311-345): the Q third (ReLU)
      goes to ``out_linearattn`` [B, tokens, N/3], the per-head ``[V | 1]^T relu(K)`` sums to ``out_vk``
      [B, heads, 33, 32] fp32; :func:`linearattn_vk_mul_q` then finishes it as in the reference;
    * ``rotary_emb`` + ``norm_q`` + ``norm_k``: RMSNorm of q / k per 128-wide head and rotary embedding
      (launch_impl.cuh:347-405), written either to ``out`` [M, N] or, head-major, to ``out_q / out_k / out_v``
      [B, heads, tokens_pad, 128] (``attn_tokens`` valid tokens per batch, padding rows zero);
      ``rotary_emb`` is the reference's packed fp32 [1, M_pad, 128] tensor (``pack_rotemb``);
    * otherwise ``out`` with optional SiLU.

    ``act_layout`` / ``out_layout`` give the memory order of the incoming / produced activation tensors.

    ``rope_cos`` / ``rope_sin`` (fp32 [S, 64], with ``norm_q`` / ``norm_k`` and ``rope_heads``) ask for the same RMSNorm +
    rotary embedding from plain tables, computed inside the GEMM's epilogue when the shape allows (else by a second
    kernel): into ``out`` [rows, 3*heads*128], or with ``rope_out = (q, k, v)`` into three token-major tensors
    [rows / S, S_total, heads*128] from token ``rope_token_offset`` on.
    """
    if poolout is not None:
        raise NotImplementedError("poolout is unused by the reference launcher as well")
    if ascales is None or wscales is None:
        raise ValueError("ascales and wscales are required")
    require_cuda_contiguous("act", act, (torch.uint8, torch.int8))
    require_cuda_contiguous("ascales", ascales, (torch.float8_e4m3fn,) if fp4 else HALF_DTYPES)
    require_cuda_contiguous("lora_act_in", lora_act_in, (torch.float32,))
    require_cuda_contiguous("out", out, HALF_DTYPES)
    if (lora_act_in is None) != (lora_up is None):
        raise ValueError("lora_act_in and lora_up must be given together")
    if lora_scales is None and lora_up is not None:
        lora_scales = [1.0] * math.ceil(lora_up.shape[1] / 16)  # nunchaku/ops/gemm.py:123-125
    if act_layout is None:
        act_layout = default_act_layout()
    dev = act.device

    M_pad = act.shape[0]
    K = act.shape[1] * 2
    prepared = cached_prepared_weights(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4)
    N = prepared.N

    if act_layout == _lib.LAYOUT_REFERENCE:
        act, ascales, lora_act_in = relayout_act(act, ascales, lora_act_in, K, fp4, _lib.LAYOUT_REFERENCE, _lib.LAYOUT_NATIVE)

    requant = qout is not None and oscales is not None
    litela = out_linearattn is not None
    rope = rotary_emb is not None
    packqkv = out_q is not None
    tmp_out = None
    if requant:
        if lora_down is None or lora_act_out is None or smooth_factor is None:
            raise ValueError("next-layer requantisation needs lora_down, lora_act_out and smooth_factor")
        activation = _lib.ACT_GELU
        M = out.shape[0] if out is not None else M_pad
        want_layout = default_act_layout() if out_layout is None else out_layout
    elif litela or (rope and packqkv):
        # these epilogues consume the projection's bf16 tile and write derived tensors only: the tile goes to a
        # scratch tensor and the row-wise kernels below finish the job
        if litela and out_vk is None:
            raise ValueError("out_linearattn needs out_vk (gemm_w4a4_launch_impl.cuh:313)")
        activation = _lib.ACT_NONE
        M = M_pad
        tmp_out = out = torch.empty(M_pad, N, dtype=prepared.half_dtype, device=dev)
    else:
        if out is None and rope_out is None:
            raise ValueError("either `out` or (`qout`, `oscales`) must be given")
        activation = _lib.ACT_SILU if fuse_silu else _lib.ACT_NONE
        M = out.numel() // out.shape[-1] if out is not None else rope_out[0].shape[0] * rope_cos.shape[0]
    if rope and (norm_q is None or norm_k is None):
        raise ValueError("rotary_emb needs norm_q and norm_k (gemm_w4a4_launch_impl.cuh:348-349)")
    if next_fp4 is None:
        next_fp4 = fp4

    # one 16-bit type per call: the weights' (as prepared), the output's, the INT4 scales' and the next layer's
    half = require_same_half_dtype(out=out, ascales=None if fp4 else ascales, smooth_factor=smooth_factor, lora_down=lora_down,
                                   oscales=None if (oscales is None or oscales.dtype == torch.float8_e4m3fn) else oscales)
    if half is None:
        half = prepared.half_dtype
    if half != prepared.half_dtype and (lora_up is not None or bias is not None or wcscales is not None or not fp4):
        raise ValueError(f"the call's tensors are {half} but the layer's parameters are {prepared.half_dtype}")

    a = prepared.args()
    a.rope_cos = None   # the struct is reused between calls
    a.dtype = dtype_code(half)
    a.act = act.data_ptr()
    a.ascales = ascales.data_ptr()
    a.lora_act_in = ptr(lora_act_in)
    a.out = ptr(out)
    a.M = M
    a.M_pad = M_pad
    a.act_unsigned = int(act_unsigned)
    a.activation = activation
    a.act_layout = _lib.LAYOUT_NATIVE
    # `out` narrower than the padded weights (the reference's actualN): the padded columns are dropped by the store
    a.N_out = out.shape[-1] if out is not None and out.shape[-1] != N else 0
    ws = None
    if requant:
        a.qout = qout.data_ptr()
        a.oscales = oscales.data_ptr()
        a.lora_act_out = lora_act_out.data_ptr()
        a.next_smooth = smooth_factor.data_ptr()
        a.next_lora_down = lora_down.data_ptr()
        a.R_next = lora_down.shape[1]
        a.out_layout = _lib.LAYOUT_NATIVE   # what the kernel writes; converted below when the caller wants the reference order
        a.next_fp4 = int(next_fp4)
    else:
        a.qout = a.oscales = a.lora_act_out = a.next_smooth = a.next_lora_down = None
        a.R_next = 0
    lib = _lib.load()
    wkey = (M_pad, a.R_next, int(requant), out is None)
    need = prepared.workspace_bytes.get(wkey)
    if need is None:
        n = ctypes.c_size_t(0)
        a.workspace = None
        a.workspace_bytes = 0
        _lib.check(lib.svdq_gemm_w4a4_workspace_bytes(prepared.tls.ref, ctypes.byref(n)))
        need = prepared.workspace_bytes[wkey] = n.value
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        a.workspace = ws.data_ptr()
        a.workspace_bytes = need
    else:
        a.workspace = None
        a.workspace_bytes = 0
    if rope and not packqkv and rope_cos is None and rotary_emb.dim() == 3 and rotary_emb.shape[2] == 128:
        # the reference's packed rotary tensor, in place on `out`: same epilogue, tables unpacked once per tensor
        from .fused import unpack_rotemb
        rope_cos, rope_sin = unpack_rotemb(rotary_emb)
        rope_heads, rope_eps, rope_out, rope_token_offset, rope = N // 384, 1e-6, None, 0, False
    if rope_cos is not None:
        if _gemm_rope_tables(a, lib, prepared, dev, out, norm_q, norm_k, rope_cos, rope_sin, rope_heads, rope_eps, rope_out,
                             rope_token_offset, M_pad, N):
            return
    with on_device(dev):
        _lib.check(lib.svdq_gemm_w4a4(prepared.tls.ref, stream_ptr(dev)))
        if requant and want_layout == _lib.LAYOUT_REFERENCE:
            co, so, lo = relayout_act(qout, oscales, lora_act_out, N, bool(next_fp4), _lib.LAYOUT_NATIVE, _lib.LAYOUT_REFERENCE)
            qout.copy_(co)
            oscales.copy_(so)
            lora_act_out.copy_(lo)
        if rope:
            from .fused import _norm_rope_packed
            _norm_rope_packed(out, norm_q, norm_k, rotary_emb, out_q, out_k, out_v, attn_tokens)
        if litela:
            from .fused import _litela_epilogue
            _litela_epilogue(tmp_out, out_vk, out_linearattn)
