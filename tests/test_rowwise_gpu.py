"""Row-wise kernels either side of the W4A4 linears against their CPU restatements."""
import pytest
import torch

from nunchaku_b200 import _lib
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


def _bf16_close(got, exp, ulps=1.0, frac=0.999):
    """all values within `ulps` bf16 steps (of the expected value) for at least `frac` of the elements, none beyond 4"""
    d = (got.float() - exp.float()).abs()
    step = exp.float().abs().clamp(min=1e-6) * 2.0 ** -7
    assert (d <= ulps * step).float().mean().item() >= frac
    assert (d <= 4 * step + 1e-6).all()


@pytest.mark.parametrize("B,S,heads", [(1, 48, 2), (3, 100, 24)])
def test_qk_norm_rope_matches_oracle(B, S, heads):
    from nunchaku_b200.ops import qk_norm_rope

    g = torch.Generator().manual_seed(B * 1000 + S)
    dim = heads * 128
    qkv = (torch.randn(B * S, 3 * dim, generator=g) * 2).to(torch.bfloat16)
    wq = (1 + 0.2 * torch.randn(128, generator=g)).to(torch.bfloat16)
    wk = (1 + 0.2 * torch.randn(128, generator=g)).to(torch.bfloat16)
    ang = torch.rand(S, 64, generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    exp = R.ref_qk_norm_rope(qkv, wq, wk, cos, sin, heads)
    got = qk_norm_rope(qkv.cuda().view(B, S, 3 * dim), wq.cuda(), wk.cuda(), cos.cuda(), sin.cuda(), heads).cpu().view(B * S, 3 * dim)
    assert torch.equal(got[:, 2 * dim:], qkv[:, 2 * dim:])          # V untouched
    _bf16_close(got[:, :2 * dim], exp[:, :2 * dim])


@pytest.mark.parametrize("B,S,C", [(2, 70, 256), (1, 333, 3072), (2, 64, 2304), (3, 50, 2240)])
def test_layernorm_modulate_matches_oracle(B, S, C):
    from nunchaku_b200.ops import layernorm_modulate

    g = torch.Generator().manual_seed(C + S)
    x = (torch.randn(B, S, C, generator=g) * 3 + 0.5).to(torch.bfloat16)
    mod = (torch.randn(B, 6 * C, generator=g) * 0.3).to(torch.bfloat16)
    shift, scale = mod[:, :C], mod[:, C:2 * C]                      # views into a wider modulation tensor
    exp = R.ref_layernorm_modulate(x, scale, shift)
    modg = mod.cuda()
    got = layernorm_modulate(x.cuda(), modg[:, C:2 * C], modg[:, :C]).cpu()
    _bf16_close(got, exp, ulps=1.0, frac=0.995)


@pytest.mark.parametrize("B,S,heads", [(1, 37, 2), (2, 1024, 72), (3, 300, 5)])
def test_litela_matches_oracle(B, S, heads):
    """ReLU linear attention: vk within fp32 summation error of the float64 oracle, the bf16 output within one bf16
    rounding of it (relative L2 <= 3e-3, no element off by more than 2 ulp of bf16 = 2^-7 relative)."""
    from nunchaku_b200.ops import litela_attention

    g = torch.Generator().manual_seed(B * 1000 + S)
    qkv = torch.randn(B, S, 3 * heads * 32, generator=g).to(torch.bfloat16)
    exp, exp_vk = R.ref_litela(qkv, heads)
    got, vk = litela_attention(qkv.cuda(), heads, return_vk=True)
    got2 = litela_attention(qkv.cuda(), heads)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.equal(got, got2)                                   # deterministic, with and without the vk output
    assert R.rel_l2(vk.cpu(), exp_vk) <= 1e-5
    g32, e32 = got.float().cpu(), exp.float()
    assert R.rel_l2(g32, e32) <= 3e-3
    assert ((g32 - e32).abs() <= 2.0 ** -7 * e32.abs() + 1e-6).all()
