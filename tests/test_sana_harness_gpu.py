"""SANA-architecture harness on the INT4 / NVFP4 W4A4 path: padded feature counts (2240 -> 2304), SiLU fused into the
expand projection, the gated quantiser input and the linear attention kernel, run end to end on random packed weights;
and the SANA layer shape against the oracle."""
import pytest
import torch

import helpers as H
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("precision", ["int4", "nvfp4"])
def test_small_sana_runs_finite_and_repeatable(precision):
    from nunchaku_b200 import _lib
    from nunchaku_b200.models.sana import SanaTransformer

    torch.manual_seed(0)
    m = SanaTransformer(dim=160, cross_heads=2, hidden=400, n_blocks=2, in_channels=32, caption_dim=96, precision=precision)
    assert len(m.w4a4_linears()) == 2 * 6
    B, Hh, Ww, T = 2, 8, 8, 20
    args = (torch.randn(B, Hh * Ww, 32, device="cuda", dtype=torch.bfloat16),
            torch.randn(B, T, 96, device="cuda", dtype=torch.bfloat16), torch.tensor([0.2, 0.9], device="cuda"))
    with torch.no_grad():
        y1 = m(*args, (Hh, Ww))
        y2 = m(*args, (Hh, Ww))
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert y1.shape == (B, Hh * Ww, 32) and torch.isfinite(y1).all() and torch.equal(y1, y2)


@pytest.mark.parametrize("fp4", [False, True])
def test_sana_layer_shape_matches_oracle(fp4):
    """One image of SANA at 1024 px: 1024 tokens, hidden 2240 against parameters padded to 2304.  The quantiser is given
    the unpadded input (K_in: missing columns read as zeros) and the GEMM an unpadded output (N_out: padded columns
    dropped); both must equal what padding with zero columns and slicing gives: codes and scales bit for bit."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops import svdq_gemm_w4a4_cuda, svdq_quantize_w4a4_act_fuse_lora_cuda

    M, K, Kp, N, Np = 1000, 2240, 2304, 2240, 2304
    xs = R.make_activations(M, K, seed=7)
    x = torch.zeros(M, Kp, dtype=torch.bfloat16)
    x[:, :K] = xs
    absmax = x.float().abs().amax(0).clamp_min(1e-3)
    lin = R.make_linear(Kp, Np, 32, fp4=fp4, x_absmax=absmax, seed=8, mode="svd", wcscales=fp4)
    m = H.to_module(lin, "cuda:0")
    q_pad = m.quantize(x.cuda())
    q_in = svdq_quantize_w4a4_act_fuse_lora_cuda(xs.cuda(), lora_down=m.proj_down, smooth=m.smooth_factor, fp4=fp4)
    for a, b in zip(q_pad, q_in):
        assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    svdq_gemm_w4a4_cuda(act=q_in[0], wgt=m.qweight, out=out, ascales=q_in[1], wscales=m.wscales, lora_act_in=q_in[2],
                        lora_up=m.proj_up, bias=m.bias, fp4=fp4, alpha=m.wtscale, wcscales=m.wcscales)
    full = m.forward_quant(*q_pad, torch.empty(M, Np, dtype=torch.bfloat16, device="cuda"))
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.equal(out, full[:, :N])
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    assert R.rel_l2(out.float().cpu(), R.ref_gemm(q, lin, M=M)[:, :N]) <= 1e-2     # tolerance of the path: relative L2 <= 1e-2
