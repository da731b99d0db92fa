"""Python wrapper of the W4A4 GEMM; same signature as ``nunchaku/ops/gemm.py:12-159``
(``svdq_gemm_w4a4_cuda``).

Weights arrive in the reference's packed order (the checkpoint format).  The sm_100a
kernel streams K-major tiles with TMA, so each layer's weights are re-tiled once
(`svdq_w4a4_prepare_weights`) and cached here, keyed by the identity of the packed
parameter tensors.
"""
from __future__ import annotations

import ctypes
import math
import weakref

import torch

from .. import _lib
from ..utils import default_act_layout, ptr, require_cuda_contiguous, stream_ptr


class PreparedWeights:
    """Device buffers holding one layer's weights in the kernel's streaming order."""

    def __init__(self, N: int, K: int, R: int, fp4: bool, device: torch.device):
        sizes = (ctypes.c_size_t * 5)()
        _lib.check(_lib.load().svdq_w4a4_prepared_bytes(N, K, R, int(fp4), sizes))
        self.N, self.K, self.R, self.fp4 = N, K, R, fp4
        self.wgt = torch.empty(sizes[0], dtype=torch.uint8, device=device)
        self.wscales = torch.empty(sizes[1], dtype=torch.uint8, device=device)
        self.lora_up = torch.empty(max(sizes[2], 16), dtype=torch.uint8, device=device)
        self.col_scale = torch.empty(sizes[3], dtype=torch.uint8, device=device)
        self.col_bias = torch.empty(sizes[4], dtype=torch.uint8, device=device)

    def as_struct(self) -> _lib.PreparedWeights:
        return _lib.PreparedWeights(
            wgt=ptr(self.wgt), wscales=ptr(self.wscales), lora_up=ptr(self.lora_up) if self.R else None,
            col_scale=ptr(self.col_scale), col_bias=ptr(self.col_bias),
        )


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
    require_cuda_contiguous("wscales", wscales, (torch.float8_e4m3fn,) if fp4 else (torch.bfloat16,))
    require_cuda_contiguous("lora_up", lora_up, (torch.bfloat16,))
    require_cuda_contiguous("bias", bias, (torch.bfloat16,))
    require_cuda_contiguous("wcscales", wcscales, (torch.bfloat16,))
    N, K = wgt.shape[0], wgt.shape[1] * 2
    R = 0 if lora_up is None else lora_up.shape[1]
    out = PreparedWeights(N, K, R, fp4, wgt.device)
    ls = None
    if lora_scales is not None:
        ls = (ctypes.c_float * len(lora_scales))(*lora_scales)
    args = _lib.WeightsArgs(
        qweight=ptr(wgt), wscales=ptr(wscales), lora_up=ptr(lora_up), bias=ptr(bias), wcscales=ptr(wcscales),
        lora_scales=ls, alpha=float(alpha), N=N, K=K, R=R, fp4=int(fp4),
    )
    st = out.as_struct()
    with torch.cuda.device(wgt.device):
        _lib.check(_lib.load().svdq_w4a4_prepare_weights(ctypes.byref(args), ctypes.byref(st), stream_ptr(wgt.device)))
    return out


_cache: dict[tuple, tuple[PreparedWeights, list]] = {}
_alpha_cache: dict[tuple, tuple[float, weakref.ref]] = {}


def _ident(t: torch.Tensor | None):
    return None if t is None else (t.data_ptr(), t._version, tuple(t.shape))


def _alpha_value(alpha) -> float:
    """``alpha`` is ``SVDQW4A4Linear.wtscale`` (a CUDA parameter) or a float.  The reference
    converts the tensor to a C++ float on every call (an implicit device sync,
    nunchaku/csrc/ops.h:33); here the value is read once per tensor version."""
    if alpha is None:
        return 1.0
    if isinstance(alpha, torch.Tensor):
        # keyed by address + version, and only valid while that very tensor object is alive: the allocator
        # hands the address of a freed one-element tensor to the next one
        key = _ident(alpha)
        hit = _alpha_cache.get(key)
        if hit is not None and hit[1]() is alpha:
            return hit[0]
        value = float(alpha.detach().float().reshape(-1)[0].item())
        if len(_alpha_cache) > 4096:
            for k in [k for k, v in _alpha_cache.items() if v[1]() is None]:
                del _alpha_cache[k]
        _alpha_cache[key] = (value, weakref.ref(alpha))
        return value
    return float(alpha)


def cached_prepared_weights(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4) -> PreparedWeights:
    a = _alpha_value(alpha)
    key = (_ident(wgt), _ident(wscales), _ident(lora_up), _ident(bias), _ident(wcscales), a,
           None if lora_scales is None else tuple(lora_scales), bool(fp4))
    hit = _cache.get(key)
    live = [t for t in (wgt, wscales, lora_up, bias, wcscales) if t is not None]
    if hit is not None and len(hit[1]) == len(live) and all(r() is t for r, t in zip(hit[1], live)):
        return hit[0]
    if lora_scales is not None and all(s == 1.0 for s in lora_scales):
        lora_scales = None
    prepared = prepare_weights(wgt, wscales, lora_up, bias, wcscales, a, lora_scales, fp4)
    refs = [weakref.ref(t) for t in live]
    _cache[key] = (prepared, refs)
    if len(_cache) > 4096:  # drop entries whose parameters are gone
        for k in [k for k, v in _cache.items() if any(r() is None for r in v[1])]:
            del _cache[k]
    return prepared


def clear_prepared_cache() -> None:
    _cache.clear()
    _alpha_cache.clear()


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
    with torch.cuda.device(codes.device):
        _lib.check(_lib.load().svdq_w4a4_relayout_act(ctypes.byref(args), stream_ptr(codes.device)))
    return co, so, lo


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
) -> None:
    """W4A4 GEMM with the fused SVDQuant epilogue; results are written in place.

    Argument meaning follows the reference.  ``qout``/``oscales`` (+ ``lora_down``,
    ``lora_act_out``, ``smooth_factor``) select the GELU + next-layer requantisation
    epilogue (gemm_w4a4_launch_impl.cuh:282-309); ``out`` the plain one with optional
    SiLU.  The attention epilogues (``norm_q``/``rotary_emb``/``out_q``..., ``out_vk``/
    ``out_linearattn``) raise NotImplementedError: both exist as kernels that run on the GEMM's bf16 output
    (``qk_norm_rope``, ``litela_attention``).  ``act_layout`` /
    ``out_layout`` give the memory order of the incoming / produced activation tensors.
    """
    if any(t is not None for t in (norm_q, norm_k, rotary_emb, out_q, out_k, out_v)):
        raise NotImplementedError("svdq_b200: the RMSNorm+RoPE / packed-QKV epilogue is not built")
    if out_vk is not None or out_linearattn is not None:
        raise NotImplementedError("svdq_b200: linear attention is not a GEMM epilogue here: write `out` and call "
                                  "nunchaku_b200.ops.litela_attention on it")
    if poolout is not None:
        raise NotImplementedError("poolout is unused by the reference launcher as well")
    if ascales is None or wscales is None:
        raise ValueError("ascales and wscales are required")
    require_cuda_contiguous("act", act, (torch.uint8, torch.int8))
    require_cuda_contiguous("ascales", ascales, (torch.float8_e4m3fn,) if fp4 else (torch.bfloat16,))
    require_cuda_contiguous("lora_act_in", lora_act_in, (torch.float32,))
    require_cuda_contiguous("out", out, (torch.bfloat16,))
    if (lora_act_in is None) != (lora_up is None):
        raise ValueError("lora_act_in and lora_up must be given together")
    if lora_scales is None and lora_up is not None:
        lora_scales = [1.0] * math.ceil(lora_up.shape[1] / 16)  # nunchaku/ops/gemm.py:123-125
    act_layout = default_act_layout() if act_layout is None else act_layout
    out_layout = default_act_layout() if out_layout is None else out_layout

    M_pad = act.shape[0]
    K = act.shape[1] * 2
    N = wgt.shape[0]
    R = 0 if lora_up is None else lora_up.shape[1]
    prepared = cached_prepared_weights(wgt, wscales, lora_up, bias, wcscales, alpha, lora_scales, fp4)

    if act_layout == _lib.LAYOUT_REFERENCE:
        act, ascales, lora_act_in = relayout_act(act, ascales, lora_act_in, K, fp4, _lib.LAYOUT_REFERENCE, _lib.LAYOUT_NATIVE)
        act_layout = _lib.LAYOUT_NATIVE

    requant = qout is not None and oscales is not None
    if requant:
        if lora_down is None or lora_act_out is None or smooth_factor is None:
            raise ValueError("next-layer requantisation needs lora_down, lora_act_out and smooth_factor")
        activation = _lib.ACT_GELU
        M = out.shape[0] if out is not None else M_pad
    else:
        if out is None:
            raise ValueError("either `out` or (`qout`, `oscales`) must be given")
        activation = _lib.ACT_SILU if fuse_silu else _lib.ACT_NONE
        M = out.shape[0]
    if next_fp4 is None:
        next_fp4 = fp4

    args = _lib.GemmArgs(
        act=ptr(act), ascales=ptr(ascales), lora_act_in=ptr(lora_act_in), w=prepared.as_struct(),
        out=ptr(out), qout=ptr(qout) if requant else None, oscales=ptr(oscales) if requant else None,
        lora_act_out=ptr(lora_act_out) if requant else None,
        next_smooth=ptr(smooth_factor) if requant else None, next_lora_down=ptr(lora_down) if requant else None,
        workspace=None, workspace_bytes=0,
        M=M, M_pad=M_pad, N=N, K=K, R=R, R_next=lora_down.shape[1] if requant else 0,
        fp4=int(fp4), act_unsigned=int(act_unsigned), activation=activation,
        act_layout=act_layout, out_layout=out_layout, next_fp4=int(next_fp4),
        # `out` narrower than the padded weights (the reference's actualN): the padded columns are dropped by the store
        N_out=out.shape[-1] if out is not None and out.shape[-1] != N else 0,
    )
    lib = _lib.load()
    ws = None
    need = ctypes.c_size_t(0)
    _lib.check(lib.svdq_gemm_w4a4_workspace_bytes(ctypes.byref(args), ctypes.byref(need)))
    if need.value:
        ws = torch.empty(need.value, dtype=torch.uint8, device=act.device)
        args.workspace = ptr(ws)
        args.workspace_bytes = need.value
    with torch.cuda.device(act.device):
        _lib.check(lib.svdq_gemm_w4a4(ctypes.byref(args), stream_ptr(act.device)))
