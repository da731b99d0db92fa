"""ctypes binding of ``oracle/_ref/libnunchaku_ref_int4.so``: the reference's own INT4 (bf16 and fp16) W4A4 kernels, built by
``python -m oracle.build_ref`` from the reference tree (test infrastructure; see ``oracle/ref_int4_shim.cu``).
All tensors are in the reference's packed orders; helpers below convert from the oracle's logical tensors."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_void_p

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "oracle", "_ref", "libnunchaku_ref_int4.so")


class QuantArgs(Structure):
    _fields_ = [("input", c_void_p), ("output", c_void_p), ("oscales", c_void_p), ("lora_down", c_void_p),
                ("lora_act_out", c_void_p), ("smooth", c_void_p), ("M", c_int), ("in_cols", c_int), ("M_pad", c_int),
                ("K_pad", c_int), ("R", c_int), ("fuse_glu", c_int), ("device", c_int), ("fp16", c_int)]


class GemmArgs(Structure):
    _fields_ = [(n, c_void_p) for n in (
        "act", "wgt", "out", "qout", "ascales", "wscales", "oscales", "lora_act_in", "lora_up", "lora_down", "lora_act_out",
        "norm_q", "norm_k", "rotary_emb", "bias", "smooth_factor", "out_vk", "out_linearattn", "out_q", "out_k", "out_v")] + [
        ("lora_scales", POINTER(c_float))] + [(n, c_int) for n in (
            "M", "M_pad", "N", "N_out", "K", "R_up", "R_down", "act_unsigned", "fuse_silu", "n_lora_scales", "batch", "heads",
            "tokens", "tokens_pad", "attn_tokens", "device", "fp16")]


_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        lib.ref_int4_quantize.argtypes = [POINTER(QuantArgs), c_void_p]
        lib.ref_int4_gemm.argtypes = [POINTER(GemmArgs), c_void_p]
        lib.ref_int4_vk_mul_q.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        if hasattr(lib, "ref_int4_quantize_wgt"):
            lib.ref_int4_quantize_wgt.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.ref_int4_last_error.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference kernel call failed: " + load().ref_int4_last_error().decode())


def _p(t):
    return None if t is None else t.data_ptr()


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def quantize(x: torch.Tensor, smooth_packed: torch.Tensor, lora_down_packed: torch.Tensor, fuse_glu: bool = False):
    """x bf16 [M, K] (or [M, 2K]); returns (codes int8 [M_pad, K/2], scales bf16 [K/64, M_pad], lora_act fp32 [M_pad, R]) in
    the reference's packed orders."""
    dev = x.device
    M, cols = x.shape
    K = cols // 2 if fuse_glu else cols
    K_pad = (K + 127) // 128 * 128
    M_pad = (M + 255) // 256 * 256
    R = lora_down_packed.shape[1]
    assert smooth_packed.numel() == K_pad and lora_down_packed.shape[0] == K_pad
    codes = torch.empty(M_pad, K_pad // 2, dtype=torch.int8, device=dev)
    scales = torch.empty(K_pad // 64, M_pad, dtype=x.dtype, device=dev)
    lora = torch.empty(M_pad, R, dtype=torch.float32, device=dev)
    a = QuantArgs(_p(x), _p(codes), _p(scales), _p(lora_down_packed), _p(lora), _p(smooth_packed), M, cols, M_pad, K_pad, R,
                  int(fuse_glu), dev.index or 0, int(x.dtype == torch.float16))
    _check(load().ref_int4_quantize(ctypes.byref(a), _stream(dev)))
    return codes, scales, lora


def gemm(act, wgt, ascales, wscales, *, out=None, qout=None, oscales=None, lora_act_in=None, lora_up=None, lora_down=None,
         lora_act_out=None, norm_q=None, norm_k=None, rotary_emb=None, bias=None, smooth_factor=None, out_vk=None,
         out_linearattn=None, out_q=None, out_k=None, out_v=None, act_unsigned=False, fuse_silu=False, attn_tokens=0):
    dev = act.device
    M_pad, K = act.shape[0], act.shape[1] * 2
    N = wgt.shape[0]
    R_up = 0 if lora_up is None else lora_up.shape[1]
    R_down = 0 if lora_down is None else lora_down.shape[1]
    ls = (c_float * max(1, R_up // 16))(*([1.0] * max(1, R_up // 16)))
    a = GemmArgs()
    for n, t in dict(act=act, wgt=wgt, out=out, qout=qout, ascales=ascales, wscales=wscales, oscales=oscales, lora_act_in=lora_act_in,
                     lora_up=lora_up, lora_down=lora_down, lora_act_out=lora_act_out, norm_q=norm_q, norm_k=norm_k,
                     rotary_emb=rotary_emb, bias=bias, smooth_factor=smooth_factor, out_vk=out_vk, out_linearattn=out_linearattn,
                     out_q=out_q, out_k=out_k, out_v=out_v).items():
        setattr(a, n, _p(t))
    a.lora_scales = ls
    a.M = out.numel() // out.shape[-1] if out is not None else M_pad
    a.M_pad, a.N, a.K = M_pad, N, K
    a.N_out = out.shape[-1] if out is not None else N
    a.R_up, a.R_down = R_up, R_down
    a.act_unsigned, a.fuse_silu, a.n_lora_scales = int(act_unsigned), int(fuse_silu), R_up // 16
    if out_vk is not None:
        a.batch, a.heads, a.tokens = out_vk.shape[0], out_vk.shape[1], out_linearattn.shape[1]
    if out_q is not None:
        a.batch, a.heads, a.tokens_pad = out_q.shape[0], out_q.shape[1], out_q.shape[2]
    a.attn_tokens = attn_tokens
    a.device = dev.index or 0
    a.fp16 = int(wscales.dtype == torch.float16)
    _check(load().ref_int4_gemm(ctypes.byref(a), _stream(dev)))


def vk_mul_q(q: torch.Tensor, vk: torch.Tensor):
    B, tokens, D = q.shape
    _check(load().ref_int4_vk_mul_q(_p(q), _p(vk), B, tokens, D // 32, q.device.index or 0, _stream(q.device)))


def has_quantize_wgt() -> bool:
    return available() and hasattr(load(), "ref_int4_quantize_wgt")


def quantize_wgt(w: torch.Tensor):
    """The reference's quantize_w4a4_wgt on a bf16 / fp16 CUDA weight [N, K] -> (packed int8 [N, K/2], packed scales [K/64, N])."""
    N, K = w.shape
    out = torch.empty(N, K // 2, dtype=torch.int8, device=w.device)
    sc = torch.empty(K // 64, N, dtype=w.dtype, device=w.device)
    _check(load().ref_int4_quantize_wgt(_p(w), _p(out), _p(sc), N, K, int(w.dtype == torch.float16), w.device.index or 0,
                                        _stream(w.device)))
    return out, sc
