"""FLUX-architecture harness: the W4A4 model (every block linear through the quantiser + 4-bit GEMM, MLPs through
fused_gelu_mlp) tracks its own bf16 master model on random weights."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("precision", ["nvfp4", "int4"])
def test_small_flux_w4a4_tracks_bf16(precision):
    from nunchaku_b200.models.flux import FluxTransformer
    from nunchaku_b200.models.linear import SVDQW4A4Linear

    torch.manual_seed(0)
    kw = dict(dim=256, heads=2, mlp_dim=1024, n_joint=1, n_single=1, in_channels=64, txt_dim=128, pooled_dim=64)
    ref = FluxTransformer(precision=None, **kw)
    q = copy.deepcopy(ref).quantize_(precision=precision, rank=32)
    lin = q.w4a4_linears()
    assert len(lin) == 8 + 4 and all(isinstance(m, SVDQW4A4Linear) for m in lin)
    B, H, W, T = 2, 8, 12, 40
    latents = torch.randn(B, H * W, 64, device="cuda", dtype=torch.bfloat16)
    text = torch.randn(B, T, 128, device="cuda", dtype=torch.bfloat16)
    pooled = torch.randn(B, 64, device="cuda", dtype=torch.bfloat16)
    t = torch.tensor([0.3, 0.7], device="cuda")
    g = torch.tensor([3.5, 3.5], device="cuda")
    with torch.no_grad():
        y_ref = ref(latents, text, pooled, t, g, (H, W))
        y_q = q(latents, text, pooled, t, g, (H, W))
        y_q2 = q(latents, text, pooled, t, g, (H, W))
    assert y_q.shape == (B, H * W, 64) and torch.isfinite(y_q).all()
    assert torch.equal(y_q, y_q2)                      # deterministic end to end
    assert _rel(y_q, y_ref) < 0.15                     # two 4-bit blocks against the bf16 masters


@pytest.mark.parametrize("precision", ["nvfp4", "int4"])
def test_random_w4a4_weights_run(precision):
    """randomize_w4a4_ (the step-timing path: random packed parameters, no SVD) gives a finite, repeatable forward."""
    from nunchaku_b200.models.flux import FluxTransformer

    torch.manual_seed(1)
    m = FluxTransformer(precision=None, dim=256, heads=2, mlp_dim=1024, n_joint=1, n_single=2, in_channels=64, txt_dim=128,
                        pooled_dim=64).randomize_w4a4_(precision, 32)
    assert len(m.w4a4_linears()) == 8 + 2 * 4
    B, H, W, T = 1, 8, 8, 32
    args = (torch.randn(B, H * W, 64, device="cuda", dtype=torch.bfloat16), torch.randn(B, T, 128, device="cuda", dtype=torch.bfloat16),
            torch.randn(B, 64, device="cuda", dtype=torch.bfloat16), torch.tensor([0.5], device="cuda"), torch.tensor([3.5], device="cuda"))
    with torch.no_grad():
        y1 = m(*args, (H, W))
        y2 = m(*args, (H, W))
    assert torch.isfinite(y1).all() and torch.equal(y1, y2)
