"""ctypes binding of ``libsvdq_b200.so`` (the C ABI declared in ``include/svdq_b200.h``).

The library is the only compute backend: if it is missing the import fails
loudly, there is no eager / CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SVDQ_B200_LIB") or os.path.join(_HERE, "libsvdq_b200.so")

SVDQ_OK = 0
SVDQ_ERR_INVALID_ARGUMENT = -1
SVDQ_ERR_UNSUPPORTED = -2
SVDQ_ERR_UNSUPPORTED_ARCH = -3
SVDQ_ERR_CUDA = -4
SVDQ_ERR_TIMEOUT = -5

LAYOUT_NATIVE = 0
LAYOUT_REFERENCE = 1

ACT_NONE = 0
ACT_SILU = 1
ACT_GELU = 2


class QuantizeArgs(Structure):
    _fields_ = [
        ("input", c_void_p),
        ("codes", c_void_p),
        ("scales", c_void_p),
        ("lora_act", c_void_p),
        ("smooth", c_void_p),
        ("lora_down", c_void_p),
        ("M", c_int32),
        ("M_pad", c_int32),
        ("K", c_int32),
        ("R", c_int32),
        ("fp4", c_int32),
        ("fuse_glu", c_int32),
        ("layout", c_int32),
        ("K_in", c_int32),
        ("dtype", c_int32),
    ]


class PreparedWeights(Structure):
    _fields_ = [
        ("wgt", c_void_p),
        ("wscales", c_void_p),
        ("lora_up", c_void_p),
        ("col_scale", c_void_p),
        ("col_bias", c_void_p),
    ]


class WeightsArgs(Structure):
    _fields_ = [
        ("qweight", c_void_p),
        ("wscales", c_void_p),
        ("lora_up", c_void_p),
        ("bias", c_void_p),
        ("wcscales", c_void_p),
        ("lora_scales", POINTER(c_float)),
        ("alpha", c_float),
        ("N", c_int32),
        ("K", c_int32),
        ("R", c_int32),
        ("fp4", c_int32),
        ("dtype", c_int32),
    ]


class GemmArgs(Structure):
    _fields_ = [
        ("act", c_void_p),
        ("ascales", c_void_p),
        ("lora_act_in", c_void_p),
        ("w", PreparedWeights),
        ("out", c_void_p),
        ("qout", c_void_p),
        ("oscales", c_void_p),
        ("lora_act_out", c_void_p),
        ("next_smooth", c_void_p),
        ("next_lora_down", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("M", c_int32),
        ("M_pad", c_int32),
        ("N", c_int32),
        ("K", c_int32),
        ("R", c_int32),
        ("R_next", c_int32),
        ("fp4", c_int32),
        ("act_unsigned", c_int32),
        ("activation", c_int32),
        ("act_layout", c_int32),
        ("out_layout", c_int32),
        ("next_fp4", c_int32),
        ("N_out", c_int32),
        ("dtype", c_int32),
        ("rope_norm_q", c_void_p),
        ("rope_norm_k", c_void_p),
        ("rope_cos", c_void_p),
        ("rope_sin", c_void_p),
        ("rope_out_q", c_void_p),
        ("rope_out_k", c_void_p),
        ("rope_out_v", c_void_p),
        ("rope_eps", c_float),
        ("rope_seq_len", c_int32),
        ("rope_heads", c_int32),
        ("rope_tokens_pad", c_int32),
        ("rope_token_offset", c_int32),
        ("rope_attn_tokens", c_int32),
    ]


class RelayoutArgs(Structure):
    _fields_ = [
        ("codes_in", c_void_p),
        ("codes_out", c_void_p),
        ("scales_in", c_void_p),
        ("scales_out", c_void_p),
        ("lora_in", c_void_p),
        ("lora_out", c_void_p),
        ("M_pad", c_int32),
        ("K", c_int32),
        ("R", c_int32),
        ("fp4", c_int32),
        ("from_layout", c_int32),
        ("to_layout", c_int32),
    ]


class NormRopeArgs(Structure):
    _fields_ = [
        ("qkv", c_void_p),
        ("weight_q", c_void_p),
        ("weight_k", c_void_p),
        ("cos", c_void_p),
        ("sin", c_void_p),
        ("rows", ctypes.c_int64),
        ("seq_len", c_int32),
        ("heads", c_int32),
        ("eps", c_float),
        ("rotary_packed", c_void_p),
        ("out_q", c_void_p),
        ("out_k", c_void_p),
        ("out_v", c_void_p),
        ("tokens_pad", c_int32),
        ("attn_tokens", c_int32),
        ("token_offset", c_int32),
        ("token_major", c_int32),
        ("dtype", c_int32),
    ]


class LnModulateArgs(Structure):
    _fields_ = [
        ("x", c_void_p),
        ("scale", c_void_p),
        ("shift", c_void_p),
        ("out", c_void_p),
        ("rows", ctypes.c_int64),
        ("rows_per_batch", ctypes.c_int64),
        ("mod_stride", ctypes.c_int64),
        ("cols", c_int32),
        ("eps", c_float),
        ("dtype", c_int32),
    ]


class GateResidualArgs(Structure):
    _fields_ = [
        ("x", c_void_p),
        ("gate", c_void_p),
        ("y", c_void_p),
        ("z", c_void_p),
        ("out", c_void_p),
        ("rows", ctypes.c_int64),
        ("rows_per_batch", ctypes.c_int64),
        ("gate_stride", ctypes.c_int64),
        ("cols", c_int32),
        ("dtype", c_int32),
    ]


class QuantizeWgtArgs(Structure):
    _fields_ = [
        ("input", c_void_p),
        ("qweight", c_void_p),
        ("wscales", c_void_p),
        ("N", c_int32),
        ("K", c_int32),
        ("dtype", c_int32),
    ]


class AttentionArgs(Structure):
    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("o_stride", ctypes.c_int64 * 3),
        ("batch", c_int32),
        ("heads", c_int32),
        ("q_len", c_int32),
        ("kv_len", c_int32),
        ("head_dim", c_int32),
        ("scale", ctypes.c_float),
        ("dtype", c_int32),
    ]


class LiteLAArgs(Structure):
    _fields_ = [
        ("qkv", c_void_p),
        ("out", c_void_p),
        ("vk", c_void_p),
        ("batches", c_int32),
        ("tokens", c_int32),
        ("heads", c_int32),
        ("eps", c_float),
        ("mode", c_int32),
        ("dtype", c_int32),
    ]


# every symbol include/svdq_b200.h declares: (restype, argtypes)
EXPORTS = {
    "svdq_quantize_w4a4_act_fuse_lora": (c_int32, [POINTER(QuantizeArgs), c_void_p]),
    "svdq_w4a4_prepared_bytes": (c_int32, [c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t)]),
    "svdq_w4a4_prepare_weights": (c_int32, [POINTER(WeightsArgs), POINTER(PreparedWeights), c_void_p]),
    "svdq_gemm_w4a4_workspace_bytes": (c_int32, [POINTER(GemmArgs), POINTER(c_size_t)]),
    "svdq_gemm_w4a4": (c_int32, [POINTER(GemmArgs), c_void_p]),
    "svdq_gemm_w4a4_static_scratch": (c_int32, [POINTER(GemmArgs), c_void_p]),
    "svdq_w4a4_relayout_act": (c_int32, [POINTER(RelayoutArgs), c_void_p]),
    "svdq_qk_norm_rope": (c_int32, [POINTER(NormRopeArgs), c_void_p]),
    "svdq_layernorm_modulate": (c_int32, [POINTER(LnModulateArgs), c_void_p]),
    "svdq_gate_residual": (c_int32, [POINTER(GateResidualArgs), c_void_p]),
    "svdq_litela": (c_int32, [POINTER(LiteLAArgs), c_void_p]),
    "svdq_attention": (c_int32, [POINTER(AttentionArgs), c_void_p]),
    "svdq_quantize_w4a4_wgt": (c_int32, [POINTER(QuantizeWgtArgs), c_void_p]),
    "svdq_device_status": (c_int32, [POINTER(c_int32), POINTER(c_int32)]),
    "svdq_last_error_string": (c_char_p, []),
    "svdq_version": (c_int32, []),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m nunchaku_b200.csrc.build` "
                "(nvcc, sm_100a). There is no fallback implementation."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class SVDQError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"svdq_b200 error {code}: {message}")
        self.code = code


def check(rc: int) -> None:
    """Map a C-ABI status to the exception the reference would raise: shape / dtype
    violations (host asserts there) become ValueError, everything else RuntimeError."""
    if rc == SVDQ_OK:
        return
    msg = load().svdq_last_error_string().decode("utf-8", "replace")
    if rc == SVDQ_ERR_INVALID_ARGUMENT:
        raise ValueError(f"svdq_b200: {msg}")
    if rc == SVDQ_ERR_UNSUPPORTED:
        raise NotImplementedError(f"svdq_b200: {msg}")
    raise SVDQError(rc, msg)


def device_status() -> tuple[int, int]:
    s, d = c_int32(0), c_int32(0)
    check(load().svdq_device_status(ctypes.byref(s), ctypes.byref(d)))
    return s.value, d.value
