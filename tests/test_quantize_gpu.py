"""Parity of the CUDA quantiser (through the C ABI) with the CPU oracle: packed 4-bit codes and
scale bytes bit-exact, low-rank activations to fp32 summation-order tolerance."""
import pytest
import torch

import helpers as H
from oracle import layouts as L
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu

LORA_RTOL = 2e-5  # fp32 accumulation over K in a different order than the fp64 oracle


def run_case(M, K, Rk, fp4, layout, x=None, seed=0):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    if x is None:
        x = R.make_activations(M, K, seed=seed + M + K)
    lin = R.make_linear(K, 128, Rk, fp4=fp4, x_absmax=x.float().abs().amax(0).clamp(min=1e-3), seed=3)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    codes, scales, lora = svdq_quantize_w4a4_act_fuse_lora_cuda(
        x.cuda(), lora_down=L.ref_pack_lora_down(lin.lora_down).cuda(), smooth=L.ref_pack_vector(lin.smooth).cuda(),
        fp4=fp4, layout=_lib.LAYOUT_NATIVE if layout == "native" else _lib.LAYOUT_REFERENCE,
    )
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    ec, es, el = H.pack_quant_out(q, layout)
    view = torch.uint8 if fp4 else torch.int16
    got = H.unpack_quant_out(codes, scales, lora, K, fp4, layout)
    H.assert_codes_match(got.codes, q)
    if q.tie is None or not q.tie.any():
        assert torch.equal(codes.cpu(), ec), "packed 4-bit codes differ from the oracle"
    assert torch.equal(scales.cpu().view(view), es.view(view)), "scale bytes differ from the oracle"
    err = (lora.cpu() - el).abs().max().item()
    tol = LORA_RTOL * max(el.abs().max().item(), 1.0) + 1e-6
    assert err <= tol, f"lora_act M={M} K={K} R={Rk} fp4={fp4} {layout}: max err {err:.3e} > {tol:.3e} ({int(((lora.cpu() - el).abs() > tol).sum())} elements)"
    return q


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("layout", ["native", "reference"])
@pytest.mark.parametrize("M,K,Rk", [(256, 128, 32), (300, 512, 32), (520, 256, 16), (256, 1024, 64), (1, 384, 48), (256, 256, 128),
                                     (300, 256, 80), (256, 384, 112), (300, 512, 160), (256, 256, 256), (70, 128, 1024)])
def test_quantize_matches_oracle(M, K, Rk, fp4, layout):
    run_case(M, K, Rk, fp4, layout)


@pytest.mark.parametrize("fp4", [True, False])
def test_quantize_headline_shapes(fp4):
    # the activations of the INT4 (M=4096, K=3072) and NVFP4 (M=4608, K=3072) workloads, and the MLP's second layer
    run_case(4096, 3072, 32, fp4, "native")
    run_case(4608, 3072, 32, fp4, "native")
    run_case(4608, 12288, 32, fp4, "native")


@pytest.mark.parametrize("fp4", [True, False])
def test_quantize_edge_values(fp4):
    """Zero rows / zero groups, negative zeros, a huge outlier that saturates the E4M3 scale,
    ties at rounding boundaries."""
    M, K = 256, 256
    g = torch.Generator().manual_seed(9)
    x = torch.randn(M, K, generator=g)
    x[3] = 0.0
    x[5, :16] = 0.0
    x[7, 16:32] = -0.0
    x[9, 40] = 3.0e4          # scale would exceed 448 -> clamps
    x[11, :64] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 8)  # E2M1 midpoints when max is 6
    x[13, :64] = torch.arange(64).float() * 0.5 - 16.0
    run_case(M, K, 32, fp4, "native", x=x.to(torch.bfloat16))
    run_case(M, K, 32, fp4, "reference", x=x.to(torch.bfloat16))


def test_quantize_deterministic():
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    x = R.make_activations(4608, 3072, seed=1).cuda()
    lin = R.make_linear(3072, 128, 32, fp4=True, seed=3)
    ld, sm = L.ref_pack_lora_down(lin.lora_down).cuda(), L.ref_pack_vector(lin.smooth).cuda()
    a = svdq_quantize_w4a4_act_fuse_lora_cuda(x, lora_down=ld, smooth=sm, fp4=True)
    b = svdq_quantize_w4a4_act_fuse_lora_cuda(x, lora_down=ld, smooth=sm, fp4=True)
    for u, v in zip(a, b):
        assert torch.equal(u.view(torch.uint8), v.view(torch.uint8))  # no atomics: bitwise repeatable


def test_relayout_round_trip():
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import relayout_act

    for fp4 in (True, False):
        x = R.make_activations(512, 256, seed=2)
        lin = R.make_linear(256, 128, 32, fp4=fp4, seed=3)
        q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
        ref = [t.cuda() for t in H.pack_quant_out(q, "reference")]
        nat = [t for t in H.pack_quant_out(q, "native")]
        got = relayout_act(*ref, 256, fp4, _lib.LAYOUT_REFERENCE, _lib.LAYOUT_NATIVE)
        for g_, e_ in zip(got, nat):
            assert torch.equal(g_.cpu().view(torch.uint8), e_.view(torch.uint8))
        back = relayout_act(*got, 256, fp4, _lib.LAYOUT_NATIVE, _lib.LAYOUT_REFERENCE)
        for g_, e_ in zip(back, ref):
            assert torch.equal(g_.view(torch.uint8), e_.view(torch.uint8))


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("M,K", [(300, 256), (1024, 2304)])
def test_quantize_fuse_glu(M, K, fp4):
    """fuse_glu (gemm_base.cuh:612-623): the input holds (value, gate) pairs and value * silu(gate) is what gets
    projected and quantised.  The kernel evaluates the sigmoid with ex2.approx / rcp.approx like the reference, the
    oracle exactly, so a gated bf16 value can differ by one ulp for a few elements.  Tolerance: the gated value v that
    the kernel quantised is checked indirectly: dequantised output within 0.6 % relative L2 of the oracle's, at
    least 99 % of the 4-bit codes and 99.5 % of the scale bytes identical, low-rank activations within 1e-3."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, 2 * K, generator=g) * 1.5).to(torch.bfloat16)
    v = (x[:, 0::2].float() * (x[:, 1::2].float() * torch.sigmoid(x[:, 1::2].float())).to(torch.bfloat16).float()).to(torch.bfloat16)
    lin = R.make_linear(K, 128, 32, fp4=fp4, x_absmax=v.float().abs().amax(0).clamp(min=1e-3), seed=3)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4, fuse_glu=True)
    codes, scales, lora = svdq_quantize_w4a4_act_fuse_lora_cuda(
        x.cuda(), lora_down=L.ref_pack_lora_down(lin.lora_down).cuda(), smooth=L.ref_pack_vector(lin.smooth).cuda(),
        fp4=fp4, fuse_glu=True, layout=_lib.LAYOUT_NATIVE,
    )
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert codes.shape == (q.codes.shape[0], K // 2)
    got = H.unpack_quant_out(codes, scales, lora, K, fp4, "native")
    assert (got.codes == q.codes).float().mean().item() >= 0.99
    view = torch.uint8 if fp4 else torch.int16
    assert (got.scales.view(view) == q.scales.view(view)).float().mean().item() >= 0.995
    assert R.rel_l2(R.dequant_act(got)[:M], R.dequant_act(q)[:M]) <= 6e-3
    assert R.rel_l2(got.lora_act[:M], q.lora_act[:M]) <= 1e-3
    assert not got.codes[M:].any()                       # rows past M are zero input: zero codes
