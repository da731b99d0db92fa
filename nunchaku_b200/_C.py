"""Stand-in for the reference's compiled extension module ``nunchaku._C`` on the W4A4 path.

The reference's Python layer reaches its kernels through two callables of a pybind submodule,
``nunchaku._C.ops.gemm_w4a4`` and ``nunchaku._C.ops.quantize_w4a4_act_fuse_lora`` (registered at
``nunchaku/csrc/pybind.cpp:108-116``, signatures ``nunchaku/csrc/ops.h:10-38,82-89``), and a handful of process-wide
knobs in ``nunchaku._C.utils`` (``pybind.cpp:118-123``).  This module offers the same names with the same positional
argument order, so the reference's own ``nunchaku/ops/{quantize,gemm,fused}.py`` and ``nunchaku/models/linear.py`` run
unmodified when ``nunchaku._C`` resolves to it (``sys.modules["nunchaku._C"] = nunchaku_b200._C`` before importing
them, or a one-line ``nunchaku/_C.py`` that re-exports this module).

Every tensor argument may be ``None`` (the reference's "invalid tensor"); results are written in place and nothing is
returned, as there.  Differences: launches go to torch's current stream on the tensors' device instead of the legacy
default stream, ``alpha`` given as a tensor is read once per layer instead of once per call, errors are Python
exceptions (``ValueError`` for what the reference asserts on) instead of ``abort()``.
"""
from __future__ import annotations

import types

import torch

from .ops.attention import attention_fp16 as _attention_fp16
from .ops.gemm import svdq_gemm_w4a4_cuda as _gemm
from .ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda as _quantize


def _gemm_w4a4(act, wgt, out, qout, ascales, wscales, oscales, poolout, lora_act_in, lora_up, lora_down, lora_act_out,
               norm_q, norm_k, rotary_emb, bias, smooth_factor, out_vk, out_linearattn, act_unsigned, lora_scales, fuse_silu,
               fp4, alpha, wcscales, out_q, out_k, out_v, attn_tokens) -> None:
    """``nunchaku::ops::gemm_w4a4`` (nunchaku/csrc/ops.h:10-80): 29 positional arguments in the reference's order."""
    _gemm(act, wgt, out, qout, ascales, wscales, oscales, poolout, lora_act_in, lora_up, lora_down, lora_act_out, norm_q,
          norm_k, rotary_emb, bias, smooth_factor, out_vk, out_linearattn, bool(act_unsigned),
          None if lora_scales is None else list(lora_scales), bool(fuse_silu), bool(fp4), alpha, wcscales, out_q, out_k, out_v,
          int(attn_tokens))


def _quantize_w4a4_act_fuse_lora(input, output, oscales, lora_down, lora_act_out, smooth, fuse_glu, fp4) -> None:
    """``nunchaku::ops::quantize_w4a4_act_fuse_lora`` (nunchaku/csrc/ops.h:82-110): the caller allocates the three
    outputs (nunchaku/ops/quantize.py:41-51) and they are written in place."""
    if output is None or oscales is None or lora_act_out is None:
        raise ValueError("output, oscales and lora_act_out must be allocated by the caller")
    _quantize(input, output, oscales, lora_down, lora_act_out, smooth, bool(fuse_glu), bool(fp4), pad_size=256)


_state = {"log_level": "info", "cuda_stack_limit": None, "memory_auto_release": True, "faster_i2f": "disabled"}


def _set_log_level(level: str) -> None:
    """Accepted and remembered; this library logs nothing (the reference forwards to spdlog)."""
    _state["log_level"] = str(level)


def _set_cuda_stack_limit(newval: int) -> None:
    """Accepted and ignored: the sm_100a kernels use no device stack (nunchaku/csrc/utils.h:9-14 calls cudaDeviceSetLimit)."""
    _state["cuda_stack_limit"] = int(newval)


def _disable_memory_auto_release() -> None:
    """Accepted and ignored: it tunes the stream-ordered allocator of the reference's own C++ tensors; all memory here is
    torch's (nunchaku/csrc/utils.h:16-23)."""
    _state["memory_auto_release"] = False


def _trim_memory() -> None:
    """The reference trims its stream-ordered pool (nunchaku/csrc/utils.h:25-32); the torch equivalent."""
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _set_faster_i2f_mode(mode: str) -> None:
    """Accepted and ignored: an sm_75-only integer-to-half trick (src/kernels/zgemm/gemm_w4a4.cu:8-16)."""
    _state["faster_i2f"] = str(mode)


ops = types.SimpleNamespace(gemm_w4a4=_gemm_w4a4, quantize_w4a4_act_fuse_lora=_quantize_w4a4_act_fuse_lora,
                            attention_fp16=_attention_fp16)
utils = types.SimpleNamespace(set_log_level=_set_log_level, set_cuda_stack_limit=_set_cuda_stack_limit,
                              disable_memory_auto_release=_disable_memory_auto_release, trim_memory=_trim_memory,
                              set_faster_i2f_mode=_set_faster_i2f_mode)
