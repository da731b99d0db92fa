"""Glue between the CPU oracle (logical tensors) and the GPU modules (packed tensors)."""
from __future__ import annotations

import torch

from oracle import layouts as L
from oracle import svdq_ref as R


def fp8(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.float8_e4m3fn)


def packed_params(lin: R.Linear) -> dict[str, torch.Tensor]:
    """The reference-packed parameter tensors of ``SVDQW4A4Linear`` for an oracle layer."""
    d = {
        "qweight": L.ref_pack_wgt_codes(lin.wcodes),
        "smooth_factor": L.ref_pack_vector(lin.smooth),
        "smooth_factor_orig": L.ref_pack_vector(lin.smooth),
        "proj_down": L.ref_pack_lora_down(lin.lora_down),
        "proj_up": L.ref_pack_lora_up(lin.lora_up),
    }
    if lin.fp4:
        d["wscales"] = fp8(L.ref_pack_wmscales(lin.wscales))
        d["wtscale"] = torch.tensor([lin.wtscale], dtype=lin.smooth.dtype)
        d["wcscales"] = L.ref_pack_vector(lin.wcscales)
    else:
        d["wscales"] = L.ref_pack_wscales(lin.wscales)
    if lin.bias is not None:
        d["bias"] = L.ref_pack_vector(lin.bias)
    return d


def to_module(lin: R.Linear, device="cuda", act_unsigned: bool = False):
    from nunchaku_b200.models import SVDQW4A4Linear

    m = SVDQW4A4Linear(
        lin.K, lin.N, rank=lin.R, bias=lin.bias is not None, precision="nvfp4" if lin.fp4 else "int4",
        act_unsigned=act_unsigned, device=device, torch_dtype=lin.smooth.dtype,
    )
    sd = packed_params(lin)
    with torch.no_grad():
        for k, v in sd.items():
            getattr(m, k).copy_(v.to(device))
    return m


def pack_quant_out(q: R.QuantOut, layout: str):
    """Oracle QuantOut -> (codes uint8 [M_pad,K/2], scales, lora_act) in 'native' or 'reference' order."""
    if layout == "native":
        codes = L.native_pack_codes(q.codes)
        scales = fp8(L.native_pack_sf(q.scales)) if q.fp4 else q.scales.contiguous()
        lora = q.lora_act.contiguous()
    else:
        codes = L.ref_pack_act_codes(q.codes)
        scales = fp8(L.ref_pack_amscales(q.scales)) if q.fp4 else L.ref_pack_ascales(q.scales)
        lora = L.ref_pack_lora_act(q.lora_act)
    return codes, scales, lora


def unpack_quant_out(codes, scales, lora, K: int, fp4: bool, layout: str) -> R.QuantOut:
    codes, scales, lora = codes.cpu(), scales.cpu(), lora.cpu()
    if layout == "native":
        c = L.native_unpack_codes(codes, K)
        s = L.native_unpack_sf(scales.view(torch.uint8)) if fp4 else scales
        la = lora
    else:
        c = L.ref_unpack_act_codes(codes, K)
        s = L.ref_unpack_amscales(scales.view(torch.uint8)) if fp4 else L.ref_unpack_ascales(scales)
        la = L.ref_unpack_lora_act(lora)
    return R.QuantOut(c, s, la, fp4)


def assert_codes_match(got: torch.Tensor, exp: R.QuantOut, rows=None, what: str = "4-bit codes") -> None:
    """``got`` (uint8 nibble values, same shape as ``exp.codes``) equals the oracle's codes, except that an element whose
    scaled value sits on a rounding tie (``exp.tie``) may take either neighbouring code: the kernels take the group
    scale's reciprocal with ``rcp.approx.ftz`` like the reference, the oracle with an exact division."""
    e, t = exp.codes, exp.tie
    if rows is not None:
        got, e, t = got[rows], e[rows], (None if t is None else t[rows])
    bad = got != e
    if t is not None:
        assert t.float().mean().item() <= 5e-2, "implausibly many rounding ties"
        bad = bad & ~t
    assert not bad.any(), f"{int(bad.sum())} {what} differ from the oracle away from rounding ties"
    if t is not None:
        d = (got.int() - e.int())[got != e]
        if exp.fp4:
            ok = ((got & 7).int() - (e & 7).int())[got != e].abs() <= 1
        else:
            ok = ((d + 8) % 16 - 8).abs() <= 1
        assert bool(ok.all()), "a tie may only move a code to its neighbour"


def module_quantize(m, x: torch.Tensor) -> "R.QuantOut":
    """Run the module's own quantiser on the GPU and return its output as an oracle ``QuantOut`` (native layout)."""
    codes, scales, lora = m.quantize(x)
    return unpack_quant_out(codes, scales, lora, x.shape[-1], m.precision == "nvfp4", "native")
