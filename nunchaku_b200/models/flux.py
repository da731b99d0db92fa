"""FLUX.1-architecture transformer built on ``SVDQW4A4Linear`` (diffusers-free).

The caller of the W4A4 path: a restatement of the block structure of
``nunchaku/models/transformers/transformer_flux_v2.py:28-392`` (``NunchakuFluxTransformerBlock``,
``NunchakuFluxSingleTransformerBlock``, ``NunchakuFluxTransformer2DModelV2``) without the diffusers
base classes, which are not installed here.  Geometry of FLUX.1-dev (``src/FluxModel.cpp:1230-1247``):
hidden 3072, 24 heads x 128, 19 joint + 38 single blocks, MLP 12288.  Per block the W4A4 linears are the
same as in the reference: fused QKV, attention out-projection, MLP fc1 (GELU + requantisation fused into
its GEMM epilogue through ``fused_gelu_mlp``) and fc2; the single block's ``proj_out`` is split into an
attention part and an MLP part (``transformer_flux_v2.py:176-183``).  AdaLN modulation, embedders, RMSNorm
of q/k, RoPE and attention itself are plain bf16 torch ops (the reference uses AWQ W4A16 GEMV and fused
epilogues for some of them; those are outside the W4A4 path).

Weights are random (there are no checkpoints offline) and quantised on the fly with
``nunchaku_b200.weights.quantize_linear``.  ``precision=None`` keeps bf16 ``nn.Linear`` layers, which gives
the model the quantised one is compared with in the tests.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.attention import attention
from ..ops.fused import fused_gelu_mlp, gate_residual, layernorm_modulate, qkv_proj_norm_rope
from ..weights import quantize_linear
from .linear import SVDQW4A4Linear
from .random_init import random_w4a4_linear


def _make_linear(in_f: int, out_f: int, precision: str | None, rank: int, device, dtype, std: float = 0.02):
    lin = nn.Linear(in_f, out_f, bias=True, device=device, dtype=dtype)
    with torch.no_grad():
        lin.weight.normal_(0.0, std)
        lin.bias.normal_(0.0, 0.02)
    if precision is None:
        return lin
    return quantize_linear(lin, None, rank=rank, precision=precision)


def _apply(lin, x: torch.Tensor) -> torch.Tensor:
    """x: [B, S, C] through either kind of linear."""
    return lin(x)


def _gated(x, gate, y, z, fused: bool):
    """x + gate[:, None] * (y (+ z)): one row-wise kernel on the W4A4 path, library ops for the bf16 twin."""
    if fused and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return gate_residual(x.contiguous(), gate, y.contiguous(), None if z is None else z.contiguous())
    return torch.addcmul(x, gate.unsqueeze(1), y if z is None else y + z)


def rope_table(ids: torch.Tensor, axes_dim=(16, 56, 56), theta: float = 10000.0):
    """FLUX rotary table: ids [S, 3] -> (cos, sin) of shape [S, head_dim/2]."""
    outs = []
    for i, d in enumerate(axes_dim):
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        ang = ids[:, i].to(torch.float64)[:, None] * freqs[None, :]
        outs.append(ang)
    ang = torch.cat(outs, dim=-1)
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, S, D]; rotates consecutive (even, odd) pairs."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.reshape(x.shape).to(x.dtype)


_LN_COLS = (256, 1024, 2304, 3072)


def _ln_mod(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, fused: bool) -> torch.Tensor:
    """layer_norm(x) * (1 + scale) + shift with scale / shift [B, C]."""
    if fused and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] in _LN_COLS:
        return layernorm_modulate(x.contiguous(), scale, shift)
    return F.layer_norm(x, x.shape[-1:]) * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class QKNorm(nn.Module):
    def __init__(self, dim: int, device, dtype):
        super().__init__()
        self.q = nn.RMSNorm(dim, eps=1e-6, device=device, dtype=dtype)
        self.k = nn.RMSNorm(dim, eps=1e-6, device=device, dtype=dtype)


# "tcgen05": this library's attention kernel for 128-wide heads (anything else falls through to the library call);
# "sdpa": torch.nn.functional.scaled_dot_product_attention everywhere, for comparison.
ATTENTION_BACKEND = {"name": "tcgen05"}


def _attention(q, k, v, heads: int, cos, sin, norm: QKNorm | None, norms=None):
    """q, k, v: [B, S, heads*D] (views with any row stride) -> [B, S, heads*D]."""
    B, S, C = q.shape
    D = C // heads
    q = q.view(B, S, heads, D).transpose(1, 2)
    k = k.view(B, S, heads, D).transpose(1, 2)
    v = v.view(B, S, heads, D).transpose(1, 2)
    if cos is not None:
        q = apply_rope(q, cos, sin)
        k = apply_rope(k, cos, sin)
    if ATTENTION_BACKEND["name"] == "tcgen05" and D == 128 and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        return attention(q, k, v)   # token-major in and out: no transposed copies
    o = F.scaled_dot_product_attention(q, k, v)
    return o.transpose(1, 2).reshape(B, S, C)


class FluxMLP(nn.Module):
    def __init__(self, dim, mlp_dim, precision, rank, device, dtype):
        super().__init__()
        self.fc1 = _make_linear(dim, mlp_dim, precision, rank, device, dtype)
        self.fc2 = _make_linear(mlp_dim, dim, precision, rank, device, dtype)

    def forward(self, x):
        # INT4 requantisation produces shifted unsigned codes whose compensation the reference folds into fc2's bias
        # offline; this random-weight harness has no such bias, so its INT4 MLP stays unfused
        if isinstance(self.fc1, SVDQW4A4Linear) and self.fc1.precision == "nvfp4":
            return fused_gelu_mlp(x, self.fc1, self.fc2)
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))


class FluxJointBlock(nn.Module):
    """Double-stream block (transformer_flux_v2.py:28-166)."""

    def __init__(self, dim, heads, mlp_dim, precision, rank, device, dtype):
        super().__init__()
        self.heads = heads
        self.mod_img = nn.Linear(dim, 6 * dim, device=device, dtype=dtype)
        self.mod_txt = nn.Linear(dim, 6 * dim, device=device, dtype=dtype)
        self.qkv_img = _make_linear(dim, 3 * dim, precision, rank, device, dtype)
        self.qkv_txt = _make_linear(dim, 3 * dim, precision, rank, device, dtype)
        self.norm_img = QKNorm(dim // heads, device, dtype)
        self.norm_txt = QKNorm(dim // heads, device, dtype)
        self.out_img = _make_linear(dim, dim, precision, rank, device, dtype)
        self.out_txt = _make_linear(dim, dim, precision, rank, device, dtype)
        self.mlp_img = FluxMLP(dim, mlp_dim, precision, rank, device, dtype)
        self.mlp_txt = FluxMLP(dim, mlp_dim, precision, rank, device, dtype)

    @staticmethod
    def _qkv(lin, norm: QKNorm, x, heads, cos=None, sin=None, out=None, token_offset=0):
        """Fused projection, then RMSNorm of q and k per head.  With (cos, sin) of this stream's rows and a W4A4
        projection the norm and the rotary embedding run inside the projection's GEMM (and the caller skips its own); with ``out`` that
        kernel writes q, k, v straight into the attention's [B, S_total, C] buffers at ``token_offset``."""
        B, S, C = x.shape
        D = C // heads
        if cos is not None and isinstance(lin, SVDQW4A4Linear) and D == 128:
            qkv = qkv_proj_norm_rope(x, lin, norm.q.weight, norm.k.weight, cos.contiguous(), sin.contiguous(), heads, eps=1e-6,
                                     out=out, token_offset=token_offset)
            if out is not None:
                return None, None, None, True
            q, k, v = qkv.chunk(3, dim=-1)
            return q, k, v, True
        qkv = _apply(lin, x)
        q, k, v = qkv.chunk(3, dim=-1)
        q = norm.q(q.reshape(B, S, heads, D)).reshape(B, S, C)
        k = norm.k(k.reshape(B, S, heads, D)).reshape(B, S, C)
        return q, k, v, False

    def forward(self, img, txt, temb, cos, sin):
        fused = isinstance(self.qkv_img, SVDQW4A4Linear)
        mi = self.mod_img(F.silu(temb)).chunk(6, dim=-1)     # each [B, dim]
        mt = self.mod_txt(F.silu(temb)).chunk(6, dim=-1)
        ni = _ln_mod(img, mi[1], mi[0], fused)
        nt = _ln_mod(txt, mt[1], mt[0], fused)
        T = txt.shape[1]
        B, S, C = img.shape
        if fused and C // self.heads == 128:
            # both streams write their q, k, v (normalised, rotated) into one set of token-major buffers: no concatenation
            qkv = torch.empty(3, B, T + S, C, dtype=img.dtype, device=img.device)
            bufs = (qkv[0], qkv[1], qkv[2])
            self._qkv(self.qkv_txt, self.norm_txt, nt, self.heads, cos[:T], sin[:T], bufs, 0)
            self._qkv(self.qkv_img, self.norm_img, ni, self.heads, cos[T:], sin[T:], bufs, T)
            attn = _attention(qkv[0], qkv[1], qkv[2], self.heads, None, None, None)
        else:
            qi, ki, vi, ri = self._qkv(self.qkv_img, self.norm_img, ni, self.heads, cos[T:], sin[T:])
            qt, kt, vt, rt = self._qkv(self.qkv_txt, self.norm_txt, nt, self.heads, cos[:T], sin[:T])
            roped = ri and rt
            attn = _attention(torch.cat([qt, qi], 1), torch.cat([kt, ki], 1), torch.cat([vt, vi], 1), self.heads,
                              None if roped else cos, None if roped else sin, None)
        at, ai = attn[:, :T], attn[:, T:]
        # gated residuals: one pass each
        img = _gated(img, mi[2], _apply(self.out_img, ai.contiguous()), None, fused)
        txt = _gated(txt, mt[2], _apply(self.out_txt, at.contiguous()), None, fused)
        ni = _ln_mod(img, mi[4], mi[3], fused)
        nt = _ln_mod(txt, mt[4], mt[3], fused)
        img = _gated(img, mi[5], self.mlp_img(ni), None, fused)
        txt = _gated(txt, mt[5], self.mlp_txt(nt), None, fused)
        return img, txt


class FluxSingleBlock(nn.Module):
    """Single-stream block (transformer_flux_v2.py:168-219): attention and MLP in parallel."""

    def __init__(self, dim, heads, mlp_dim, precision, rank, device, dtype):
        super().__init__()
        self.heads = heads
        self.mod = nn.Linear(dim, 3 * dim, device=device, dtype=dtype)
        self.qkv = _make_linear(dim, 3 * dim, precision, rank, device, dtype)
        self.norm = QKNorm(dim // heads, device, dtype)
        self.attn_out = _make_linear(dim, dim, precision, rank, device, dtype)
        self.mlp = FluxMLP(dim, mlp_dim, precision, rank, device, dtype)

    def forward(self, x, temb, cos, sin):
        fused = isinstance(self.qkv, SVDQW4A4Linear)
        m = self.mod(F.silu(temb)).chunk(3, dim=-1)
        n = _ln_mod(x, m[1], m[0], fused)
        q, k, v, roped = FluxJointBlock._qkv(self.qkv, self.norm, n, self.heads, cos, sin)
        a = _attention(q, k, v, self.heads, None if roped else cos, None if roped else sin, None)
        return _gated(x, m[2], _apply(self.attn_out, a.contiguous()), self.mlp(n), fused)


class FluxTransformer(nn.Module):
    """FLUX.1-dev geometry by default; every size can be shrunk for tests."""

    def __init__(self, dim=3072, heads=24, mlp_dim=12288, n_joint=19, n_single=38, in_channels=64, txt_dim=4096,
                 pooled_dim=768, precision: str | None = "nvfp4", rank=32, axes_dim=(16, 56, 56),
                 device="cuda", dtype=torch.bfloat16):
        super().__init__()
        self.dim, self.heads, self.axes_dim = dim, heads, tuple(axes_dim)
        assert sum(axes_dim) == dim // heads
        kw = dict(device=device, dtype=dtype)
        self.x_embedder = nn.Linear(in_channels, dim, **kw)
        self.context_embedder = nn.Linear(txt_dim, dim, **kw)
        self.time_mlp = nn.Sequential(nn.Linear(256, dim, **kw), nn.SiLU(), nn.Linear(dim, dim, **kw))
        self.guidance_mlp = nn.Sequential(nn.Linear(256, dim, **kw), nn.SiLU(), nn.Linear(dim, dim, **kw))
        self.pooled_mlp = nn.Sequential(nn.Linear(pooled_dim, dim, **kw), nn.SiLU(), nn.Linear(dim, dim, **kw))
        self.joint = nn.ModuleList([FluxJointBlock(dim, heads, mlp_dim, precision, rank, device, dtype) for _ in range(n_joint)])
        self.single = nn.ModuleList([FluxSingleBlock(dim, heads, mlp_dim, precision, rank, device, dtype) for _ in range(n_single)])
        self.norm_out = nn.Linear(dim, 2 * dim, **kw)
        self.proj_out = nn.Linear(dim, in_channels, **kw)
        with torch.no_grad():   # keep the residual stream tame with random weights
            for mod in self.modules():
                if isinstance(mod, nn.Linear):
                    mod.weight.normal_(0.0, 0.02)
                    if mod.bias is not None:
                        mod.bias.zero_()

    @staticmethod
    def _sinusoid(t: torch.Tensor, dim: int = 256) -> torch.Tensor:
        half = dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
        ang = t.float()[:, None] * freqs[None, :]
        return torch.cat([ang.cos(), ang.sin()], dim=-1)

    @torch.no_grad()
    def quantize_(self, precision: str = "nvfp4", rank: int = 32):
        """Replace every bf16 ``nn.Linear`` of the blocks that the reference runs as W4A4 by its SVDQuant version."""
        names = ("qkv_img", "qkv_txt", "out_img", "out_txt", "qkv", "attn_out", "fc1", "fc2")
        for mod in list(self.modules()):
            for n in names:
                child = getattr(mod, n, None)
                if isinstance(child, nn.Linear):
                    setattr(mod, n, quantize_linear(child, None, rank=rank, precision=precision))
        return self

    @torch.no_grad()
    def randomize_w4a4_(self, precision: str = "nvfp4", rank: int = 32, seed: int = 0):
        """Replace the block linears by W4A4 layers with RANDOM packed parameters (no SVD, no calibration): random 4-bit
        codes, one constant group scale sized so that weights look like N(0, 0.02), small random low-rank factors.
        For step timing at full size, where quantising 12 B master weights on the CPU would take hours."""
        g = torch.Generator(device="cuda").manual_seed(seed)
        names = ("qkv_img", "qkv_txt", "out_img", "out_txt", "qkv", "attn_out", "fc1", "fc2")
        for mod in list(self.modules()):
            for n in names:
                child = getattr(mod, n, None)
                if not isinstance(child, nn.Linear):
                    continue
                q = random_w4a4_linear(child.in_features, child.out_features, rank, precision, True, g, child.weight.device,
                                       child.weight.dtype)
                setattr(mod, n, q)
        return self

    def w4a4_linears(self):
        return [m for m in self.modules() if isinstance(m, SVDQW4A4Linear)]

    def forward(self, latents, text, pooled, timestep, guidance, img_hw: tuple[int, int]):
        """latents [B, S_img, C_in], text [B, S_txt, txt_dim], pooled [B, pooled_dim], timestep/guidance [B]."""
        dt = latents.dtype
        img = self.x_embedder(latents)
        txt = self.context_embedder(text)
        temb = (self.time_mlp(self._sinusoid(timestep * 1000).to(dt)) + self.guidance_mlp(self._sinusoid(guidance * 1000).to(dt))
                + self.pooled_mlp(pooled))
        H, W = img_hw
        ids_img = torch.zeros(H * W, 3, device=latents.device)
        ids_img[:, 1] = torch.arange(H, device=latents.device).repeat_interleave(W)
        ids_img[:, 2] = torch.arange(W, device=latents.device).repeat(H)
        ids = torch.cat([torch.zeros(text.shape[1], 3, device=latents.device), ids_img], 0)
        cos, sin = rope_table(ids, self.axes_dim)
        for blk in self.joint:
            img, txt = blk(img, txt, temb, cos, sin)
        x = torch.cat([txt, img], dim=1)
        for blk in self.single:
            x = blk(x, temb, cos, sin)
        x = x[:, text.shape[1]:]
        sc, sh = self.norm_out(F.silu(temb)).unsqueeze(1).chunk(2, dim=-1)
        x = F.layer_norm(x, x.shape[-1:]) * (1 + sc) + sh
        return self.proj_out(x)
