"""CPU restatement of the SVDQuant W4A4 linear arithmetic (test infrastructure, never shipped).

All tensors here are *logical* (unpacked, row-major); ``oracle.layouts`` turns
them into reference or native memory order.  Functions cite the reference code
they follow by file:line (paths inside the nunchaku tree).

Rounding model.  Every ``half_t`` operation of the reference is a bf16
round-to-nearest-even of the exact result.  ``__fdividef`` and
``rcp.approx.ftz`` (gemm_utils.cuh:258-262,329-344) are modelled as correctly
rounded fp32 division / reciprocal.  A group whose absolute maximum is zero has
``scale = 0``; the reference then multiplies by ``rcp(0) = inf`` and converts a
NaN, here (and in the CUDA kernels of this repository) the reciprocal of a zero
scale is defined as 0 so that such a group gets all-zero codes.  The dequantised
value (0) is the same either way.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from . import fmt

F32 = torch.float32
BF16 = torch.bfloat16
F16 = torch.float16
HALF_TYPES = (BF16, F16)   # the reference's half_t: GEMMConfig_W4A4_BF16 / _FP16 (gemm_base.cuh:29-54)

# fp32 compile-time constants of the reference (gemm_w4a4.cuh:91-93,435-441)
RCP6 = torch.tensor(1.0, dtype=F32) / torch.tensor(6.0, dtype=F32)
RCP7 = torch.tensor(1.0, dtype=F32) / torch.tensor(7.0, dtype=F32)
RCP15 = torch.tensor(1.0, dtype=F32) / torch.tensor(15.0, dtype=F32)
INT4_UNSIGNED_SHIFT = 0.171875  # gemm_w4a4_launch_impl.cuh:286-294


def ceil_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclasses.dataclass
class QuantOut:
    codes: torch.Tensor      # uint8 [M_pad, K], one nibble value per element
    scales: torch.Tensor     # NVFP4: uint8 e4m3 bytes [K/16, M_pad]; INT4: bf16 [K/64, M_pad]
    lora_act: torch.Tensor   # fp32 [M_pad, R]
    fp4: bool
    unsigned: bool = False
    tie: torch.Tensor | None = None   # bool [M_pad, K]: the scaled value sits on (or within 1e-5 of) a rounding tie


def _silu_bf16(y: torch.Tensor) -> torch.Tensor:
    """gemm_utils.cuh:321-327: (T)(float(x) * sigmoid(float(x)))."""
    yf = y.to(F32)
    return (yf * torch.sigmoid(yf)).to(y.dtype)


def gelu_f32(x: torch.Tensor) -> torch.Tensor:
    """gemm_utils.cuh:305-319: x * (0.5 + 0.5 * tanh(0.79788456 * (x + 0.044715 x^3)))."""
    x = x.to(F32)
    return x * (0.5 + 0.5 * torch.tanh(0.79788456 * (x + 0.044715 * x * x * x)))


def group_quantize(v: torch.Tensor, *, fp4: bool, unsigned: bool = False):
    """Group-quantise an already smoothed bf16 tensor ``v`` [rows, K].

    Follows quantize_w4a4_fp4_from_fpsum_warp (gemm_w4a4.cuh:85-187) and
    quantize_w4a4_from_fpsum_warp (gemm_w4a4.cuh:429-523).
    Returns (codes uint8 [rows, K], scales [K/G, rows], tie bool [rows, K]).

    The reference takes the reciprocal of the group scale with ``rcp.approx.ftz`` (gemm_utils.cuh:259-263), which this
    restatement models as the exact fp32 reciprocal.  The two differ by at most one unit in the last place, which can
    change a code only where ``v * rscale`` lies on a rounding tie; since bf16 values have 8-bit mantissas such exact
    ties are common (a few in 10^4 elements).  ``tie`` flags the elements within 1e-5 (relative) of a tie: there the
    code is "either neighbour", everywhere else it is pinned.
    """
    assert v.dtype in HALF_TYPES
    rows, K = v.shape
    G = 16 if fp4 else 64
    vf = v.to(F32).reshape(rows, K // G, G)
    amax = vf.abs().amax(dim=2)  # exact in bf16
    if fp4:
        scale = torch.minimum(amax * RCP6, torch.tensor(448.0))
        stored = fmt.e4m3_encode(scale)
    else:
        scale = amax * (RCP15 if unsigned else RCP7)
        stored = scale.to(v.dtype)
    rscale = torch.where(scale == 0, torch.zeros_like(scale), 1.0 / scale)
    q = vf * rscale.unsqueeze(2)
    codes = fmt.e2m1_encode(q) if fp4 else fmt.int4_encode(q, unsigned)
    aq = q.abs().to(torch.float64)
    if fp4:   # midpoints of the E2M1 grid {0, .5, 1, 1.5, 2, 3, 4, 6}
        mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float64)
        tie = ((aq.unsqueeze(-1) - mids).abs() <= 1e-5 * mids).any(-1)
    else:
        tie = ((aq - aq.floor()) - 0.5).abs() <= 1e-5 * aq.clamp(min=1.0)
    return codes.reshape(rows, K), stored.t().contiguous(), tie.reshape(rows, K)


def ref_quantize(
    x: torch.Tensor,
    smooth: torch.Tensor,
    lora_down: torch.Tensor | None,
    *,
    fp4: bool,
    fuse_glu: bool = False,
    pad_size: int = 256,
) -> QuantOut:
    """quantize_w4a4_fuse_lora_kernel (gemm_w4a4.cuh:1097-1184).

    x         bf16 [M, K]  ([M, 2K] interleaved (value, gate) pairs when fuse_glu)
    smooth    bf16 [K]     logical order
    lora_down bf16 [R, K]  logical order (the unpacked ``proj_down``)
    """
    assert x.dtype in HALF_TYPES and smooth.dtype == x.dtype
    HT = x.dtype
    M = x.shape[0]
    if fuse_glu:  # gemm_base.cuh:612-623: pack[j] = raw[j].x * silu(raw[j].y), both in bf16
        v = (x[:, 0::2].to(F32) * _silu_bf16(x[:, 1::2]).to(F32)).to(HT)
    else:
        v = x
    K = v.shape[1]
    M_pad = ceil_to(M, pad_size)
    vp = torch.zeros(M_pad, K, dtype=HT)
    vp[:M] = v
    # LoRA down on the un-smoothed tile (lora.cuh:243-353), fp32 accumulation
    if lora_down is not None:
        lora_act = (vp.to(torch.float64) @ lora_down.to(torch.float64).t()).to(F32)
    else:
        lora_act = torch.zeros(M_pad, 0, dtype=F32)
    # EpilogueQuantize (gemm_w4a4.cuh:930-1043) with shift_value = 0: bf16 add of +0, then h2div
    # (fp16: the reference's half division is rcp.approx(b) * a rounded once, cuda_fp16.hpp __hdiv; the exact quotient used
    # here can differ from it only within 2^-23 of a rounding boundary of the result)
    vs = (vp.to(F32) + 0.0).to(HT)
    vs = (vs.to(F32) / smooth.to(F32).unsqueeze(0)).to(HT)
    codes, scales, tie = group_quantize(vs, fp4=fp4, unsigned=False)
    return QuantOut(codes, scales, lora_act, fp4, False, tie)


def dequant_act(q: QuantOut) -> torch.Tensor:
    rows, K = q.codes.shape
    if q.fp4:
        val = fmt.e2m1_decode(q.codes)
        s = fmt.e4m3_decode(q.scales).t()  # [rows, K/16]
        return (val.reshape(rows, K // 16, 16) * s.unsqueeze(2)).reshape(rows, K)
    val = fmt.int4_decode(q.codes, q.unsigned)
    s = q.scales.to(F32).t()
    return (val.reshape(rows, K // 64, 64) * s.unsqueeze(2)).reshape(rows, K)


@dataclasses.dataclass
class Linear:
    """One SVDQuant W4A4 linear with logical (unpacked) parameters."""

    K: int
    N: int
    R: int
    fp4: bool
    wcodes: torch.Tensor          # uint8 [N, K] nibble values
    wscales: torch.Tensor         # NVFP4: uint8 e4m3 [K/16, N]; INT4: bf16 [K/64, N]
    smooth: torch.Tensor          # bf16 [K]
    lora_down: torch.Tensor       # bf16 [R, K]
    lora_up: torch.Tensor         # bf16 [N, R]
    bias: torch.Tensor | None     # bf16 [N]
    wtscale: float = 1.0          # NVFP4 per-tensor weight scale ("alpha")
    wcscales: torch.Tensor | None = None  # NVFP4 per-channel scale, bf16 [N]

    def dequant_weight(self) -> torch.Tensor:
        """fp32 [N, K]; includes ``wtscale`` but not ``wcscales``."""
        if self.fp4:
            val = fmt.e2m1_decode(self.wcodes)
            s = fmt.e4m3_decode(self.wscales).t()
            w = (val.reshape(self.N, self.K // 16, 16) * s.unsqueeze(2)).reshape(self.N, self.K)
            return w * self.wtscale
        val = fmt.int4_decode(self.wcodes, False)
        s = self.wscales.to(F32).t()
        return (val.reshape(self.N, self.K // 64, 64) * s.unsqueeze(2)).reshape(self.N, self.K)


def ref_gemm(
    q: QuantOut,
    lin: Linear,
    *,
    M: int | None = None,
    act: str | None = None,
    lora_scales: list[float] | None = None,
    use_lora: bool = True,
) -> torch.Tensor:
    """The "math" oracle of gemm_w4a4: dequantise, fp32 matmul, epilogue in fp32.

    Order of the fused epilogue (gemm_w4a4_launch_impl.cuh:172-420):
    acc*alpha -> *wcscale + bias (gemm_base.cuh:710-781) -> + LoRA-up
    (lora.cuh:110-241) -> GELU | SiLU.  Returns fp32 [M, N] (not rounded to bf16).
    """
    M = q.codes.shape[0] if M is None else M
    a = dequant_act(q)[:M]
    y = a @ lin.dequant_weight().t()
    if lin.wcscales is not None:
        y = y * lin.wcscales.to(F32).unsqueeze(0)
    if lin.bias is not None:
        y = y + lin.bias.to(F32).unsqueeze(0)
    if use_lora and lin.R > 0:
        la = q.lora_act[:M]
        if lora_scales is not None:
            sc = torch.tensor(lora_scales, dtype=F32).repeat_interleave(16)[: lin.R]
            la = la * sc.unsqueeze(0)
        y = y + la @ lin.lora_up.to(F32).t()
    if act == "gelu":
        y = gelu_f32(y)
    elif act == "silu":
        y = y * torch.sigmoid(y)
    return y


def ref_requantize(
    y: torch.Tensor,
    nxt: Linear,
    *,
    M_pad: int,
    unsigned: bool,
) -> QuantOut:
    """Next-layer requantisation fused into the GEMM epilogue
    (gemm_w4a4_launch_impl.cuh:282-309, gemm_w4a4.cuh:930-1043, lora.cuh:243-353):
    LoRA-down on the activated value, then (+shift) / smooth_next, group-quantise.
    ``y`` is the activated GEMM output in fp32 [M, N]; it is rounded to bf16 first,
    as the reference's accumulator tile is bf16 at that point."""
    M, N = y.shape
    HT = nxt.smooth.dtype
    yb = torch.zeros(M_pad, N, dtype=HT)
    yb[:M] = y.to(F32).clamp(-65504.0, 65504.0).to(HT) if HT == F16 else y.to(HT)
    lora_act = (yb.to(torch.float64) @ nxt.lora_down.to(torch.float64).t()).to(F32)
    shift = INT4_UNSIGNED_SHIFT if unsigned else 0.0
    v = (yb.to(F32) + shift).to(HT)
    v = (v.to(F32) / nxt.smooth.to(F32).unsqueeze(0)).to(HT)
    codes, scales, tie = group_quantize(v, fp4=nxt.fp4, unsigned=unsigned)
    return QuantOut(codes, scales, lora_act, nxt.fp4, unsigned, tie)


# ---------------------------------------------------------------------------
# Synthetic SVDQuant problems (the reference has no quantiser; its checkpoints
# come from the external DeepCompressor project).
# ---------------------------------------------------------------------------
def make_activations(M: int, K: int, seed: int = 0, outlier_frac: float = 0.01, outlier_mul: float = 20.0, dtype=BF16):
    """bf16 [M, K] ~ N(0,1) with a fraction of channels scaled up (outliers)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=F32)
    n_out = max(1, math.ceil(outlier_frac * K))
    cols = torch.randperm(K, generator=g)[:n_out]
    x[:, cols] *= outlier_mul
    return x.to(dtype)


def quantize_weight(res: torch.Tensor, fp4: bool, dtype=BF16):
    """Residual fp32 [N, K] -> (codes uint8 [N,K], scales [K/G, N], wtscale)."""
    N, K = res.shape
    if fp4:
        amax_t = res.abs().max().item()
        wtscale = float(torch.tensor(max(amax_t / (6.0 * 448.0), 1e-12), dtype=dtype).item())  # the module stores it in its 16-bit type
        g = res.reshape(N, K // 16, 16)
        s = g.abs().amax(dim=2) / (6.0 * wtscale)
        sb = fmt.e4m3_encode(s)
        sd = fmt.e4m3_decode(sb) * wtscale
        q = g / torch.where(sd == 0, torch.ones_like(sd), sd).unsqueeze(2)
        codes = fmt.e2m1_encode(q).reshape(N, K)
        return codes, sb.t().contiguous(), wtscale
    g = res.reshape(N, K // 64, 64)
    s = (g.abs().amax(dim=2) / 7.0).to(dtype)
    sf = s.to(F32)
    q = g / torch.where(sf == 0, torch.ones_like(sf), sf).unsqueeze(2)
    codes = fmt.int4_encode(q, False).reshape(N, K)
    return codes, s.t().contiguous(), 1.0


def make_linear(
    K: int,
    N: int,
    R: int,
    *,
    fp4: bool,
    x_absmax: torch.Tensor | None = None,
    seed: int = 0,
    mode: str = "literal",
    bias: bool = True,
    w_std: float = 0.02,
    wcscales: bool = False,
    dtype=BF16,
) -> Linear:
    """Random-init SVDQuant linear.

    ``mode='literal'``: weights ~N(0, w_std) with their rank-R SVD component
    removed, low-rank factors drawn independently ~N(0, 0.02).
    ``mode='svd'``: low-rank factors are the removed SVD component, so the layer
    approximates ``x @ W.T + b`` of the bf16 master weight (returned as ``.master``).
    """
    g = torch.Generator().manual_seed(seed + 1000003)
    W = torch.randn(N, K, generator=g, dtype=F32) * w_std
    if x_absmax is None:
        x_absmax = torch.ones(K)
    w_absmax = W.abs().amax(dim=0).clamp(min=1e-8)
    smooth = torch.sqrt(x_absmax.to(F32).clamp(min=1e-8) / w_absmax).clamp(min=1e-4).to(dtype)
    What = W * smooth.to(F32).unsqueeze(0)
    if R > 0:
        if min(N, K) <= 1024:
            U, S, Vh = torch.linalg.svd(What, full_matrices=False)
            U, S, V = U[:, :R], S[:R], Vh[:R].t()
        else:
            torch.manual_seed(seed)
            U, S, V = torch.svd_lowrank(What, q=R + 8, niter=2)
            U, S, V = U[:, :R], S[:R], V[:, :R]
        low = (U * S) @ V.t()
    else:
        low = torch.zeros_like(What)
    res = What - low
    wcodes, wscales, wtscale = quantize_weight(res, fp4, dtype)
    if mode == "literal":
        lora_down = (torch.randn(R, K, generator=g) * 0.02).to(dtype)
        lora_up = (torch.randn(N, R, generator=g) * 0.02).to(dtype)
    else:
        lora_up = (U * S).to(dtype)
        lora_down = (V.t() / smooth.to(F32).unsqueeze(0)).to(dtype)
    b = (torch.randn(N, generator=g) * 0.02).to(dtype) if bias else None
    wc = None
    if fp4:
        wc = (1.0 + 0.25 * torch.rand(N, generator=g)).to(dtype) if wcscales else torch.ones(N, dtype=dtype)
    lin = Linear(K, N, R, fp4, wcodes, wscales, smooth, lora_down, lora_up, b, wtscale, wc)
    lin.master = W  # type: ignore[attr-defined]
    return lin


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.to(torch.float64)
    b = b.to(torch.float64)
    return float((a - b).norm() / b.norm().clamp(min=1e-30))


# ---------------------------------------------------------------------------
# Row-wise steps either side of the linears
# ---------------------------------------------------------------------------
def ref_qk_norm_rope(qkv: torch.Tensor, w_q: torch.Tensor, w_k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                     heads: int, eps: float = 1e-6) -> torch.Tensor:
    """EpilogueRMSNormRope (src/kernels/zgemm/epilogues.cuh:330-405) on a bf16 [rows, 3*heads*128] QKV output:
    per head of the Q and K thirds ``coef = rsqrt(sum(float(y)^2)/128 + eps)``, ``v = float(y) * (coef * float(w))``,
    pairs (2p, 2p+1) rotated by (cos, sin)[row % S, p] in fp32, one rounding to the input's 16-bit type.  V is untouched.
    cos, sin: fp32 [S, 64]."""
    rows, C = qkv.shape
    dim = heads * 128
    assert C == 3 * dim
    S = cos.shape[0]
    out = qkv.clone()
    pos = torch.arange(rows) % S
    c, s = cos[pos].to(F32)[:, None, :], sin[pos].to(F32)[:, None, :]          # [rows, 1, 64]
    for which, w in ((0, w_q), (1, w_k)):
        y = qkv[:, which * dim:(which + 1) * dim].to(F32).view(rows, heads, 128)
        coef = torch.rsqrt((y * y).sum(-1, keepdim=True) / 128.0 + eps)
        v = y * (coef * w.to(F32)[None, None, :])
        a, b = v[..., 0::2], v[..., 1::2]
        r = torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(rows, dim)
        out[:, which * dim:(which + 1) * dim] = r.to(qkv.dtype)
    return out


def ref_layernorm_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """bf16 [B, S, C]: layer_norm without affine (fp32 statistics, result rounded to bf16, as the library call it
    replaces does), then ``* (1 + scale[b]) + shift[b]`` in fp32 with one rounding."""
    xf = x.to(F32)
    mean = xf.mean(-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    n = ((xf - mean) * torch.rsqrt(var + eps)).to(x.dtype).to(F32)
    return (n * (1.0 + scale.to(F32)[:, None, :]) + shift.to(F32)[:, None, :]).to(x.dtype)


def ref_litela(qkv: torch.Tensor, heads: int, eps: float = 1e-6):
    """ReLU linear attention on a fused QKV output [B, S, 3*heads*32] (bf16), columns [Q | (K_h, V_h) per head]
    (EpilogueLiteLA + vk_mul_q_kernel, src/kernels/zgemm/epilogues.cuh:552-761):
    vk[b,h,r,c] = sum_t V[t,r] relu(K[t,c]) (r < 32), vk[b,h,32,c] = sum_t relu(K[t,c]);
    o = relu(Q) @ vk^T; out = bf16(o[:32] / (o[32] + eps)).  Sums in float64 (the order of the fp32 sums on the GPU is
    an implementation choice); returns (out bf16 [B, S, heads*32], vk float32 [B, heads, 33, 32])."""
    B, S, C = qkv.shape
    D = heads * 32
    assert C == 3 * D
    q = qkv[..., :D].double().clamp_min(0).view(B, S, heads, 32)
    kv = qkv[..., D:].double().view(B, S, heads, 64)
    k, v = kv[..., :32].clamp_min(0), kv[..., 32:]
    v1 = torch.cat([v, torch.ones(B, S, heads, 1, dtype=torch.float64)], dim=-1)       # [B,S,H,33]
    vk = torch.einsum("bshr,bshc->bhrc", v1, k)                                         # [B,H,33,32]
    o = torch.einsum("bshc,bhrc->bshr", q, vk.float().double())                         # [B,S,H,33]
    out = (o[..., :32].float() / (o[..., 32:].float() + eps)).to(qkv.dtype)
    return out.reshape(B, S, D), vk.float()


def ref_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, round_p: bool = True) -> torch.Tensor:
    """Softmax attention per (batch, head) on 16-bit q [B, H, Tq, D], k, v [B, H, Tkv, D] as the reference's kernel states it
    (src/kernels/zgemm/attention.cuh:226-330, launcher attention.cu:10-96): S = q k^T in fp32, the scale folded with log2(e)
    into an exp2 (``cuda_exp2(fmaf(val, scale, -rowmax_scaled))``), the row sum taken from the fp32 exponentials, the
    exponentials rounded to the 16-bit type for the product with v, fp32 accumulation, one division by the row sum and one
    rounding at the end.  The order of the block-wise running maximum is an implementation choice (it only moves the
    rounding point of P by a power of two); here the row maximum is global.  Parity unpinned: the reference's tests hold no
    vectors for this kernel; tests/test_oracle_arith.py pins this function to float64 softmax loops.  Returns [B, Tq, H*D] in
    q's dtype."""
    B, H, Tq, D = q.shape
    s = (q.double() @ k.double().transpose(-1, -2)).float() * (scale * 1.4426950408889634)
    p = torch.exp2(s - s.amax(dim=-1, keepdim=True))
    l = p.double().sum(-1, keepdim=True)
    if round_p:
        p = p.to(q.dtype).float()
    o = (p.double() @ v.double()) / l
    return o.float().to(q.dtype).transpose(1, 2).reshape(B, Tq, H * D)


def ref_quantize_wgt_int4(w: torch.Tensor):
    """The reference's INT4 weight quantiser (quantize_w4a4_wgt_kernel + quantize_w4a4_warp,
    src/kernels/zgemm/gemm_w4a4.cuh:661-689,527-620) on a bf16 weight [N, K]: per row and group of 64, all in bf16,
    ``scale = max|w| / 7``, ``rscale = 7 / max|w|``, ``code = sat_s4(rint(bf16(rscale * w)))`` (round to nearest even; a zero
    group gives inf * 0 = NaN -> 0).  Returns logical (codes uint8 nibbles [N, K], scales bf16 [K/64, N]).  bf16 only: the
    reference's fp16 division is the approximate-reciprocal ``__hdiv``, which only the kernel itself reproduces."""
    assert w.dtype == BF16
    N, K = w.shape
    g = w.reshape(N, K // 64, 64)
    m = g.float().abs().amax(dim=2).to(BF16)
    seven = torch.tensor(7.0, dtype=BF16)
    scale = m / seven                      # bf16 division: the fp32 quotient rounded once
    rscale = seven / m                     # inf for a zero group
    h = (rscale.unsqueeze(2) * g)          # bf16 product, rounded once; inf * 0 = NaN
    q = torch.nan_to_num(h.float(), nan=0.0, posinf=7.0, neginf=-8.0).round().clamp(-8, 7).to(torch.int32)
    codes = (q & 0xF).to(torch.uint8).reshape(N, K)
    return codes, scale.t().contiguous()
