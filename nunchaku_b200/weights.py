"""Weight-side tooling: quantise a bf16/fp32 master weight the SVDQuant way and pack the
result into the parameter layout of :class:`nunchaku_b200.models.SVDQW4A4Linear`.

The reference ships no quantiser (its checkpoints come from the external DeepCompressor
project); it only ships the packer (``nunchaku/lora/flux/packer.py:187-398``), whose memory
orders are restated here with plain reshape/permute so that layers built from random or
real master weights are byte-compatible with reference checkpoints.  Everything here is
torch tensor code that runs on the tensors' device (CPU or CUDA); it is offline tooling,
not part of the per-step hot path.
"""
from __future__ import annotations

import torch

E2M1_MAX = 6.0
E4M3_MAX = 448.0


# --------------------------------------------------------------------------- number formats
def e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 codes (uint8, bit 3 = sign), round-to-nearest-even, saturating."""
    a = v.abs().to(torch.float32)
    # thresholds between {0, .5, 1, 1.5, 2, 3, 4, 6}; ties go to the code with an even mantissa
    mag = (a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
    mag += (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8) + (a > 5.0).to(torch.uint8)
    return mag | (torch.signbit(v).to(torch.uint8) << 3)


def int4_codes(v: torch.Tensor) -> torch.Tensor:
    return (torch.round(v).clamp(-8, 7).to(torch.int32) & 0xF).to(torch.uint8)


# --------------------------------------------------------------------------- packers
def _pack_nibbles(nib: torch.Tensor) -> torch.Tensor:
    nib = nib.reshape(-1, 2)
    return (nib[:, 0] | (nib[:, 1] << 4)).to(torch.uint8)


def pack_weight_codes(codes: torch.Tensor) -> torch.Tensor:
    """uint8 nibble values [N, K] -> int8 [N, K/2] in the order of ``pack_weight``
    (packer.py:187-239): [N/128][K/64][n-tile 8][g 8][t 4][half 2][kh 2][8 nibbles]."""
    N, K = codes.shape
    assert N % 128 == 0 and K % 128 == 0
    c = codes.reshape(N // 128, 8, 2, 8, K // 64, 2, 4, 8)       # bn nt half g bk kh t j
    c = c.permute(0, 4, 1, 3, 6, 2, 5, 7).contiguous()           # bn bk nt g t half kh j
    return _pack_nibbles(c).view(torch.int8).reshape(N, K // 2)


def pack_vector(v: torch.Tensor) -> torch.Tensor:
    """bias / smooth / wcscales [N] -> order of ``pack_scale(..., group_size=-1)``
    (packer.py:241-301): within each 128 block, n = a*16 + b*8 + c*2 + d is stored at
    a*16 + c*4 + b*2 + d."""
    N = v.numel()
    assert N % 128 == 0
    return v.reshape(N // 128, 8, 2, 4, 2).permute(0, 1, 3, 2, 4).contiguous().reshape(N)


def pack_int4_wscales(s: torch.Tensor) -> torch.Tensor:
    """[K/64, N] -> same nominal shape, order [N/128][K/64][a][c][b][d] (packer.py:241-301)."""
    G, N = s.shape
    p = s.reshape(G, N // 128, 8, 2, 4, 2).permute(1, 0, 2, 4, 3, 5).contiguous()
    return p.reshape(G, N)


def pack_nvfp4_wscales(s: torch.Tensor) -> torch.Tensor:
    """float8_e4m3fn [K/16, N] -> same nominal shape, order of ``pack_micro_scale``
    (packer.py:303-360): [N/128][K/64][d 8][c 4][s 4][kg 4], n = s*32 + c*8 + d."""
    G16, N = s.shape
    b = s.view(torch.uint8).reshape(G16 // 4, 4, N // 128, 4, 4, 8)   # bk kg bn s c d
    b = b.permute(2, 0, 5, 4, 3, 1).contiguous()
    return b.reshape(G16, N).view(torch.float8_e4m3fn)


def pack_lora_up(w: torch.Tensor) -> torch.Tensor:
    """[N, R] -> order of ``pack_lowrank_weight(down=False)`` (packer.py:362-398)."""
    N, R = w.shape
    p = w.reshape(N // 16, 2, 8, R // 16, 2, 4, 2)                     # cp nh g rp kh t e
    return p.permute(0, 3, 2, 5, 1, 4, 6).contiguous().reshape(N, R)


def pack_lora_down(w: torch.Tensor) -> torch.Tensor:
    """logical [R, K] -> packed ``proj_down`` with nominal shape [K, R]
    (``pack_lowrank_weight(down=True)``, packer.py:362-398)."""
    R, K = w.shape
    p = w.reshape(R // 16, 2, 8, K // 16, 2, 4, 2)                     # rp nh g cp kh t e
    return p.permute(3, 0, 2, 5, 1, 4, 6).contiguous().reshape(K, R)


# --------------------------------------------------------------------------- SVDQuant-lite
@torch.no_grad()
def svdquant_state_dict(
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    x_absmax: torch.Tensor | None,
    rank: int = 32,
    precision: str = "nvfp4",
    dtype: torch.dtype = torch.bfloat16,
    extra_bias: torch.Tensor | None = None,
    random_lowrank_std: float | None = None,
) -> dict[str, torch.Tensor]:
    """Quantise ``weight`` [N, K] into the packed parameters of ``SVDQW4A4Linear``.

    smooth = sqrt(max|x| / max|w|) per input channel; W_hat = W * smooth; the top-``rank``
    singular component of W_hat goes to the low-rank branch (``proj_up = U S``,
    ``proj_down = diag(1/smooth) V`` because the kernel applies it to the un-smoothed
    activation, gemm_w4a4.cuh:1159-1182); the residual is group-quantised (INT4 group 64,
    symmetric, or NVFP4 group 16 with E4M3 scales and a per-tensor ``wtscale``).
    With ``random_lowrank_std`` the SVD component is still removed from the residual but the
    stored low-rank factors are drawn ~N(0, std) instead (a synthetic-benchmark layer that does
    not approximate ``weight``).
    """
    N, K = weight.shape
    W = weight.to(torch.float32)
    dev = W.device
    if x_absmax is None:
        x_absmax = torch.ones(K, device=dev)
    w_absmax = W.abs().amax(dim=0).clamp(min=1e-8)
    smooth = torch.sqrt(x_absmax.to(dev, torch.float32).clamp(min=1e-8) / w_absmax).clamp(min=1e-4).to(dtype)
    What = W * smooth.to(torch.float32).unsqueeze(0)
    if rank > 0:
        if min(N, K) <= 512:
            U, S, Vh = torch.linalg.svd(What, full_matrices=False)
            U, S, V = U[:, :rank], S[:rank], Vh[:rank].t()
        else:
            U, S, V = torch.svd_lowrank(What, q=rank + 8, niter=2)
            U, S, V = U[:, :rank], S[:rank], V[:, :rank]
        up = (U * S)
        res = What - up @ V.t()
        down = (V.t() / smooth.to(torch.float32).unsqueeze(0))
        if random_lowrank_std is not None:
            up = torch.randn_like(up) * random_lowrank_std
            down = torch.randn_like(down) * random_lowrank_std
    else:
        res = What
    sd: dict[str, torch.Tensor] = {}
    if precision == "nvfp4":
        wtscale = (res.abs().max() / (E2M1_MAX * E4M3_MAX)).clamp(min=1e-12).to(dtype)
        g = res.reshape(N, K // 16, 16)
        s8 = (g.abs().amax(dim=2) / (E2M1_MAX * wtscale.float())).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
        sd_eff = s8.to(torch.float32) * wtscale.float()
        codes = e2m1_codes(g / torch.where(sd_eff == 0, torch.ones_like(sd_eff), sd_eff).unsqueeze(2)).reshape(N, K)
        sd["wscales"] = pack_nvfp4_wscales(s8.t().contiguous())
        sd["wtscale"] = wtscale.reshape(1)
        sd["wcscales"] = torch.ones(N, dtype=dtype, device=dev)
    elif precision == "int4":
        g = res.reshape(N, K // 64, 64)
        s = (g.abs().amax(dim=2) / 7.0).to(dtype)
        sf = s.to(torch.float32)
        codes = int4_codes(g / torch.where(sf == 0, torch.ones_like(sf), sf).unsqueeze(2)).reshape(N, K)
        sd["wscales"] = pack_int4_wscales(s.t().contiguous())
    else:
        raise ValueError(f"Invalid precision: {precision}")
    sd["qweight"] = pack_weight_codes(codes)
    sd["smooth_factor"] = pack_vector(smooth)
    sd["smooth_factor_orig"] = sd["smooth_factor"].clone()
    if rank > 0:
        sd["proj_up"] = pack_lora_up(up.to(dtype))
        sd["proj_down"] = pack_lora_down(down.to(dtype))
    b = None if bias is None else bias.to(torch.float32)
    if extra_bias is not None:
        b = extra_bias.to(torch.float32) if b is None else b + extra_bias.to(torch.float32)
    if b is not None:
        sd["bias"] = pack_vector(b.to(dtype))
    return sd


@torch.no_grad()
def quantize_linear(
    linear: torch.nn.Linear,
    x_absmax: torch.Tensor | None = None,
    rank: int = 32,
    precision: str = "nvfp4",
    act_unsigned: bool = False,
):
    """``nn.Linear`` -> ``SVDQW4A4Linear`` on the same device."""
    from .models.linear import SVDQW4A4Linear

    m = SVDQW4A4Linear.from_linear(linear, rank=rank, precision=precision, act_unsigned=act_unsigned)
    sd = svdquant_state_dict(linear.weight, linear.bias, x_absmax, rank, precision, linear.weight.dtype)
    for k, v in sd.items():
        getattr(m, k).copy_(v)
    return m
