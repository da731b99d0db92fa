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


def test_sana_layer_shape_int4_matches_oracle():
    """One image of SANA at 1024 px: 1024 tokens, hidden 2240 padded to 2304 with zero columns, INT4 group 64."""
    M, K, Kp, N = 1024, 2240, 2304, 2304
    x = torch.zeros(M, Kp, dtype=torch.bfloat16)
    x[:, :K] = R.make_activations(M, K, seed=7)
    absmax = x.float().abs().amax(0).clamp_min(1e-3)
    lin = R.make_linear(Kp, N, 32, fp4=False, x_absmax=absmax, seed=8, mode="svd")
    m = H.to_module(lin, "cuda:0")
    y = m(x.cuda().view(1, M, Kp)).float().cpu().view(M, N)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    assert R.rel_l2(y, R.ref_gemm(q, lin, M=M)) <= 1e-2     # tolerance of the path: relative L2 <= 1e-2
