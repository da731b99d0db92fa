"""Number-format helpers of the oracle (test infrastructure, never shipped).

Rounding model (reference: src/kernels/zgemm/gemm_utils.cuh:206-264):
  * ``cvt.rn.satfinite.e2m1x2.f32``  -> :func:`e2m1_encode` (round to nearest,
    ties to even code, saturate to +-6, the sign of a zero result is kept).
  * ``cvt.rn.satfinite.e4m3x2.f32``  -> :func:`e4m3_encode` (inputs are already
    clamped to <= 448 at gemm_w4a4.cuh:134-135, so torch's non-saturating cast
    is exact for them).
  * ``cvt.rni.s32.f32`` + ``cvt.pack.sat.{s4,u4}`` -> :func:`int4_encode`.
"""
from __future__ import annotations

import torch

# value of each E2M1 magnitude code 0..7
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)
# decision thresholds between neighbouring magnitudes; a value exactly on a
# threshold goes to the code with an even mantissa bit (RN-even):
#   0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0
_E2M1_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32)
_E2M1_TIE_UP = torch.tensor([False, True, False, True, False, True, False])


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """fp32 tensor -> uint8 nibble codes (bit 3 = sign, bits 0..2 = magnitude)."""
    v = v.to(torch.float32)
    a = v.abs()
    mag = torch.zeros_like(a, dtype=torch.int32)
    for mid, up in zip(_E2M1_MID.tolist(), _E2M1_TIE_UP.tolist()):
        mag += (a >= mid).to(torch.int32) if up else (a > mid).to(torch.int32)
    mag = torch.where(torch.isnan(a), torch.full_like(mag, 7), mag)
    sign = torch.signbit(v) & ~torch.isnan(v)
    return (mag | (sign.to(torch.int32) << 3)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    code = code.to(torch.int64)
    val = E2M1_VALUES[code & 7]
    return torch.where((code & 8) != 0, -val, val)


def e4m3_encode(v: torch.Tensor) -> torch.Tensor:
    """fp32 (0 <= v <= 448) -> uint8 E4M3 byte, round-to-nearest-even."""
    return v.to(torch.float32).clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


def int4_encode(v: torch.Tensor, unsigned: bool) -> torch.Tensor:
    """fp32 -> nibble codes: round-half-even, NaN -> 0, saturate to s4 / u4."""
    v = torch.nan_to_num(v.to(torch.float32), nan=0.0, posinf=1e9, neginf=-1e9)
    q = torch.round(v)  # torch.round is half-to-even
    q = q.clamp(0, 15) if unsigned else q.clamp(-8, 7)
    return (q.to(torch.int32) & 0xF).to(torch.uint8)


def int4_decode(code: torch.Tensor, unsigned: bool) -> torch.Tensor:
    c = code.to(torch.int32)
    if not unsigned:
        c = torch.where(c >= 8, c - 16, c)
    return c.to(torch.float32)


def bf16_round(v: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 and return it as fp32."""
    return v.to(torch.bfloat16).to(torch.float32)
