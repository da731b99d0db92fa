"""W4A4 layers with random packed parameters, for timing and plumbing checks where no master weight is quantised:
uniform random 4-bit codes, one constant group scale sized so that the weights look like N(0, 0.02), smoothing
factors of one, N(0, 0.02) low-rank factors.  (Layers that approximate a given bf16 weight come from
``nunchaku_b200.weights.quantize_linear``.)"""
from __future__ import annotations

import torch

from .linear import SVDQW4A4Linear


@torch.no_grad()
def random_w4a4_linear(in_features: int, out_features: int, rank: int = 32, precision: str = "nvfp4", bias: bool = True,
                       generator: torch.Generator | None = None, device="cuda", dtype=torch.bfloat16,
                       bias_std: float = 0.0, int4_scale: float = 0.005) -> SVDQW4A4Linear:
    q = SVDQW4A4Linear(in_features, out_features, rank=rank, bias=bias, precision=precision, torch_dtype=dtype, device=device)
    g = generator
    q.qweight.copy_(torch.randint(-128, 128, q.qweight.shape, generator=g, device=device, dtype=torch.int16).to(torch.int8))
    if precision == "nvfp4":
        q.wscales.copy_(torch.full(q.wscales.shape, 2.0 ** -7, device=device).to(torch.float8_e4m3fn))
    else:
        q.wscales.fill_(int4_scale)
    q.smooth_factor.fill_(1.0)
    q.smooth_factor_orig.fill_(1.0)
    q.proj_down.copy_(torch.randn(q.proj_down.shape, generator=g, device=device) * 0.02)
    q.proj_up.copy_(torch.randn(q.proj_up.shape, generator=g, device=device) * 0.02)
    if bias:
        if bias_std:
            q.bias.copy_(torch.randn(q.bias.shape, generator=g, device=device) * bias_std)
        else:
            q.bias.zero_()
    return q
