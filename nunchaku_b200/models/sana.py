"""SANA-1.6B-architecture linear DiT built on the W4A4 path (diffusers-free).

The second caller of the path: a restatement of the block structure of ``src/SanaModel.cpp:13-380``
(``SanaLinearAttention``, ``MultiHeadCrossAttention``, ``SanaGLUMBConv``, ``SanaLinearTransformerBlock``, ``SanaModel``).
Geometry of SANA-1.6B: hidden 2240 = 70 heads x 32 for the ReLU linear attention, 20 x 112 for cross attention, 20 blocks,
GLUMBConv width 5600 (2.5 x), 1024 px = 32 x 32 latent tokens of 32 channels.  Per block the W4A4 linears are the
reference's: ``qkv_proj`` (its output feeds the linear attention kernel), ``out_proj``, the cross attention's
``q_linear`` and ``out_proj``, ``inverted_conv`` (SiLU fused into its GEMM epilogue) and ``point_conv`` (its quantiser
gates the (value, gate) pairs: ``fuse_glu``).  The depthwise 3 x 3 convolution, cross attention (torch SDPA), the
``kv_linear`` of the caption and the modulation are plain bf16 torch ops, as they are outside the W4A4 path.
``precision=None`` builds the same model from bf16 ``nn.Linear`` masters (the twin the quantised model is compared
with in the tests); ``quantize_`` turns such a model into the W4A4 one.

Padding as in the reference (``src/Linear.cpp:92-93``, ``SanaModel.cpp:15``): feature counts are rounded up to 128 for
the 4-bit tensors (2240 -> 2304, 2 x 5600 -> 2 x 5632); activations keep their real width: the quantiser reads the missing
columns as zeros and the GEMM does not store the padded output columns.  Weights are random packed W4A4 parameters: this module is for
step timing and for checking that the call sequence runs; there are no checkpoints offline.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.fused import gate_residual, layernorm_modulate, litela_attention
from ..ops.gemm import svdq_gemm_w4a4_cuda
from ..ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda
from .linear import SVDQW4A4Linear
from .random_init import random_w4a4_linear


def _pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def _random_w4a4(in_f: int, out_f: int, rank: int, precision: str, bias: bool, g: torch.Generator, device) -> SVDQW4A4Linear:
    return random_w4a4_linear(in_f, out_f, rank, precision, bias, g, device)


class PaddedW4A4(nn.Module):
    """A W4A4 linear whose logical feature counts are not multiples of 128: the quantiser reads the missing input columns
    as zeros and the GEMM's store drops the padded output columns (``K_in`` / ``N_out`` of the C ABI).
    With ``precision=None`` it holds the bf16 master ``nn.Linear`` instead (same call interface, plain torch arithmetic):
    the model the quantised one is compared with; :meth:`quantize_` turns it into the W4A4 layer."""

    def __init__(self, in_f, out_f, rank, precision, bias, g, device, keep_out_pad: bool = False, dtype=torch.bfloat16):
        super().__init__()
        self.in_f, self.out_f, self.keep_out_pad, self.rank = in_f, out_f, keep_out_pad, rank
        self.lin = None
        self.master = None
        if precision is None:
            self.master = nn.Linear(in_f, out_f, bias=bias, device=device, dtype=dtype)
        else:
            self.lin = _random_w4a4(_pad128(in_f), _pad128(out_f), rank, precision, bias, g, device)

    @torch.no_grad()
    def quantize_(self, precision: str):
        """bf16 master -> SVDQuant W4A4 layer with feature counts padded to 128 (zero rows / columns)."""
        from ..weights import quantize_linear

        m = self.master
        ip, op = _pad128(self.in_f), _pad128(self.out_f)
        padded = nn.Linear(ip, op, bias=m.bias is not None, device=m.weight.device, dtype=m.weight.dtype)
        padded.weight.zero_()
        padded.weight[: self.out_f, : self.in_f] = m.weight
        if m.bias is not None:
            padded.bias.zero_()
            padded.bias[: self.out_f] = m.bias
        self.lin = quantize_linear(padded, None, rank=self.rank, precision=precision)
        self.master = None
        return self

    def forward(self, x: torch.Tensor, fuse_silu: bool = False, fuse_glu: bool = False) -> torch.Tensor:
        """x: [B, S, in_f] (or already padded; [B, S, 2*in_pad] of (value, gate) pairs with fuse_glu)."""
        if self.master is not None:
            if fuse_glu:
                x = (x[..., 0::2].float() * F.silu(x[..., 1::2].float())).to(x.dtype)
            y = self.master(x[..., : self.in_f])
            return F.silu(y) if fuse_silu else y
        lin = self.lin
        B, S, C = x.shape
        q, s, la = svdq_quantize_w4a4_act_fuse_lora_cuda(
            x.reshape(B * S, C), lora_down=lin.proj_down, smooth=lin.smooth_factor, fp4=lin.precision == "nvfp4", fuse_glu=fuse_glu)
        n_out = lin.out_features if self.keep_out_pad else self.out_f
        out = torch.empty(B * S, n_out, dtype=x.dtype, device=x.device)
        svdq_gemm_w4a4_cuda(act=q, wgt=lin.qweight, out=out, ascales=s, wscales=lin.wscales, lora_act_in=la, lora_up=lin.proj_up,
                            bias=lin.bias, fp4=lin.precision == "nvfp4", alpha=lin.wtscale, wcscales=lin.wcscales,
                            fuse_silu=fuse_silu)
        return out.view(B, S, n_out)


def _litela_torch(qkv: torch.Tensor, heads: int, eps: float = 1e-6) -> torch.Tensor:
    """ReLU linear attention in plain torch (fp32), column order as the kernel's: [Q | (K_h, V_h) per head]."""
    B, S, C = qkv.shape
    D = heads * 32
    q = qkv[..., :D].float().clamp_min(0).view(B, S, heads, 32)
    kv = qkv[..., D:].float().view(B, S, heads, 64)
    k, v = kv[..., :32].clamp_min(0), kv[..., 32:]
    v1 = torch.cat([v, torch.ones_like(v[..., :1])], dim=-1)
    vk = torch.einsum("bshr,bshc->bhrc", v1, k)
    o = torch.einsum("bshc,bhrc->bshr", q, vk)
    return (o[..., :32] / (o[..., 32:] + eps)).to(qkv.dtype).reshape(B, S, D)


class SanaLinearAttention(nn.Module):
    """SanaModel.cpp:13-106."""

    def __init__(self, dim, rank, precision, g, device):
        super().__init__()
        self.dim, self.dim_pad = dim, _pad128(dim)
        self.heads = self.dim_pad // 32
        self.qkv_proj = PaddedW4A4(dim, 3 * self.dim_pad, rank, precision, False, g, device)
        self.out_proj = PaddedW4A4(self.dim_pad, dim, rank, precision, True, g, device)

    def forward(self, x):
        qkv = self.qkv_proj(x)                                   # [B, S, 3 * dim_pad]
        if self.qkv_proj.master is not None:
            return self.out_proj(_litela_torch(qkv, self.heads))
        return self.out_proj(litela_attention(qkv.contiguous(), self.heads))


class SanaCrossAttention(nn.Module):
    """SanaModel.cpp:138-190."""

    def __init__(self, dim, heads, rank, precision, g, device, dtype):
        super().__init__()
        self.heads = heads
        self.q_linear = PaddedW4A4(dim, dim, rank, precision, True, g, device)
        self.kv_linear = nn.Linear(dim, 2 * dim, device=device, dtype=dtype)
        self.out_proj = PaddedW4A4(dim, dim, rank, precision, True, g, device)

    def forward(self, x, cond):
        B, S, C = x.shape
        D = C // self.heads
        q = self.q_linear(x).reshape(B, S, self.heads, D).transpose(1, 2)
        kv = self.kv_linear(cond).view(B, cond.shape[1], 2, self.heads, D)
        k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, C))


class SanaGLUMBConv(nn.Module):
    """SanaModel.cpp:190-213: 1x1 expand (+SiLU) -> depthwise 3x3 -> gate (in the next quantiser) -> 1x1 project."""

    def __init__(self, dim, hidden, rank, precision, g, device, dtype):
        super().__init__()
        self.hidden_pad = _pad128(hidden)
        self.inverted_conv = PaddedW4A4(dim, 2 * self.hidden_pad, rank, precision, True, g, device)
        self.depth_conv = nn.Conv2d(2 * self.hidden_pad, 2 * self.hidden_pad, 3, padding=1, groups=2 * self.hidden_pad,
                                    device=device, dtype=dtype).to(memory_format=torch.channels_last)
        self.point_conv = PaddedW4A4(self.hidden_pad, dim, rank, precision, False, g, device)

    def forward(self, x, H, W):
        B, S, _ = x.shape
        y = self.inverted_conv(x, fuse_silu=True)                # [B, S, 2 * hidden_pad]
        y = self.depth_conv(y.view(B, H, W, -1).permute(0, 3, 1, 2))      # channels-last in and out
        y = y.permute(0, 2, 3, 1).reshape(B, S, -1)
        return self.point_conv(y, fuse_glu=True)


def _ln_mod(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, fused: bool = True) -> torch.Tensor:
    """layer_norm(x, eps 1e-6) * (1 + scale) + shift with scale / shift [B, C]: one row-wise kernel for the widths it is built for."""
    if fused and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] in (256, 1024, 2240, 2304, 3072):
        return layernorm_modulate(x.contiguous(), scale, shift, eps=1e-6)
    return F.layer_norm(x, x.shape[-1:], eps=1e-6) * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


def _gated(x, gate, y, fused: bool):
    """x + gate[:, None] * y (gate None = 1): one row-wise kernel on the W4A4 path, library ops for the bf16 twin."""
    if fused and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return gate_residual(x.contiguous(), gate, y.contiguous())
    return x + y if gate is None else x + gate.unsqueeze(1) * y


class SanaBlock(nn.Module):
    """SanaModel.cpp:215-320."""

    def __init__(self, dim, cross_heads, hidden, rank, precision, g, device, dtype):
        super().__init__()
        self.scale_shift_table = nn.Parameter(torch.randn(6, dim, device=device, dtype=dtype) * 0.02, requires_grad=False)
        self.attn = SanaLinearAttention(dim, rank, precision, g, device)
        self.cross_attn = SanaCrossAttention(dim, cross_heads, rank, precision, g, device, dtype)
        self.ff = SanaGLUMBConv(dim, hidden, rank, precision, g, device, dtype)

    def forward(self, x, cond, t6, H, W):
        B, S, C = x.shape
        m = (self.scale_shift_table[None] + t6.view(B, 6, C)).unbind(1)   # shift, scale, gate (attention), shift, scale, gate (MLP)
        fused = self.attn.qkv_proj.master is None
        n = _ln_mod(x, m[1], m[0], fused)
        x = _gated(x, m[2], self.attn(n), fused)
        x = _gated(x, None, self.cross_attn(x, cond), fused)
        n = _ln_mod(x, m[4], m[3], fused)
        return _gated(x, m[5], self.ff(n, H, W), fused)


class SanaTransformer(nn.Module):
    """SANA-1.6B geometry by default; every size can be shrunk for tests."""

    def __init__(self, dim=2240, cross_heads=20, hidden=5600, n_blocks=20, in_channels=32, caption_dim=2304,
                 precision="int4", rank=32, seed=0, device="cuda", dtype=torch.bfloat16):
        super().__init__()
        g = torch.Generator(device=device).manual_seed(seed)
        kw = dict(device=device, dtype=dtype)
        self.dim = dim
        self.patch_embed = nn.Linear(in_channels, dim, **kw)
        self.caption_proj = nn.Sequential(nn.Linear(caption_dim, dim, **kw), nn.GELU(approximate="tanh"), nn.Linear(dim, dim, **kw))
        self.time_mlp = nn.Sequential(nn.Linear(256, dim, **kw), nn.SiLU(), nn.Linear(dim, dim, **kw))
        self.adaln_single = nn.Linear(dim, 6 * dim, **kw)
        self.blocks = nn.ModuleList([SanaBlock(dim, cross_heads, hidden, rank, precision, g, device, dtype) for _ in range(n_blocks)])
        self.final_table = nn.Parameter(torch.randn(2, dim, **kw) * 0.02, requires_grad=False)
        self.proj_out = nn.Linear(dim, in_channels, **kw)
        with torch.no_grad():
            for mod in self.modules():
                if isinstance(mod, nn.Linear):
                    mod.weight.normal_(0.0, 0.02)
                    if mod.bias is not None:
                        mod.bias.zero_()
                elif isinstance(mod, nn.Conv2d):
                    mod.weight.normal_(0.0, 0.1)
                    mod.bias.zero_()

    def w4a4_linears(self):
        return [m for m in self.modules() if isinstance(m, SVDQW4A4Linear)]

    @torch.no_grad()
    def quantize_(self, precision: str = "int4"):
        """Turn every bf16 master projection of the blocks (a model built with ``precision=None``) into its W4A4 layer."""
        for mod in self.modules():
            if isinstance(mod, PaddedW4A4) and mod.master is not None:
                mod.quantize_(precision)
        return self

    def forward(self, latents, caption, timestep, img_hw: tuple[int, int]):
        """latents [B, H*W, C_in], caption [B, T, caption_dim], timestep [B]."""
        dt = latents.dtype
        half = 128
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=latents.device, dtype=torch.float32) / half)
        ang = timestep.float()[:, None] * 1000.0 * freqs[None, :]
        temb = self.time_mlp(torch.cat([ang.cos(), ang.sin()], dim=-1).to(dt))
        t6 = self.adaln_single(F.silu(temb))
        x = self.patch_embed(latents)
        cond = self.caption_proj(caption)
        H, W = img_hw
        for blk in self.blocks:
            x = blk(x, cond, t6, H, W)
        sh, sc = (self.final_table[None] + temb[:, None]).unbind(1)
        x = F.layer_norm(x, (self.dim,), eps=1e-6) * (1 + sc.unsqueeze(1)) + sh.unsqueeze(1)
        return self.proj_out(x)
