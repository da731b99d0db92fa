from .fused import (fused_gelu_mlp, gate_residual, fused_qkv_norm_rottary, layernorm_modulate, linearattn_vk_mul_q, litela_attention,
                    qk_norm_rope, qkv_proj_norm_rope)
from .attention import attention, attention_fp16
from .gemm import svdq_gemm_w4a4_cuda
from .quantize import svdq_quantize_w4a4_act_fuse_lora_cuda, svdq_quantize_w4a4_wgt

__all__ = ["svdq_quantize_w4a4_act_fuse_lora_cuda", "svdq_quantize_w4a4_wgt", "svdq_gemm_w4a4_cuda", "fused_gelu_mlp", "fused_qkv_norm_rottary",
           "qk_norm_rope", "qkv_proj_norm_rope", "layernorm_modulate", "gate_residual", "litela_attention", "linearattn_vk_mul_q", "attention", "attention_fp16"]
