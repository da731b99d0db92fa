"""Row-wise kernels either side of the W4A4 linears against their CPU restatements."""
import pytest
import torch

import helpers as H
from nunchaku_b200 import _lib
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


def _bf16_close(got, exp, ulps=1.0, frac=0.999):
    """all values within `ulps` bf16 steps (of the expected value) for at least `frac` of the elements, none beyond 4"""
    d = (got.float() - exp.float()).abs()
    step = exp.float().abs().clamp(min=1e-6) * 2.0 ** -7
    assert (d <= ulps * step).float().mean().item() >= frac
    assert (d <= 4 * step + 1e-6).all()


def _f16_close(got, exp, ulps=1.0, frac=0.999):
    """as _bf16_close with fp16's step (2^-10 relative)"""
    d = (got.float() - exp.float()).abs()
    step = exp.float().abs().clamp(min=1e-6) * 2.0 ** -10
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


@pytest.mark.parametrize("B,S,heads,split,dtype", [(2, 64, 2, False, torch.bfloat16), (1, 320, 4, True, torch.bfloat16),
                                                       (3, 96, 2, True, torch.bfloat16),
                                                       (2, 50, 2, True, torch.bfloat16),   # not a shape of the fused epilogue (second kernel)
                                                       (2, 96, 2, True, torch.float16), (1, 64, 2, False, torch.float16)])
def test_qkv_projection_with_norm_rope_in_the_gemm_epilogue(B, S, heads, split, dtype):
    """RMSNorm + rotary embedding inside the QKV GEMM's epilogue (svdq_gemm_args.rope_*) against (a) the same projection
    followed by the row-wise kernel and (b) the oracle on the GEMM's own bf16 tile.  The two GPU paths differ only in the
    order of the 128 additions of the sum of squares, which can move a result by one bf16 ulp now and then."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops import qk_norm_rope, qkv_proj_norm_rope

    C = heads * 128
    torch.manual_seed(S + heads)
    close = _bf16_close if dtype == torch.bfloat16 else _f16_close
    x = R.make_activations(B * S, C, seed=S, dtype=dtype)
    lin = R.make_linear(C, 3 * C, 32, fp4=True, x_absmax=x.float().abs().amax(0), seed=S + 1, mode="svd", wcscales=True, dtype=dtype)
    m = H.to_module(lin)
    wq = (1.0 + 0.1 * torch.randn(128)).to(dtype).cuda()
    wk = (1.0 + 0.1 * torch.randn(128)).to(dtype).cuda()
    ang = torch.rand(S, 64) * 6.28
    cos, sin = ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous()
    xg = x.cuda().view(B, S, C)
    tile = m(xg)                                                   # plain projection: the bf16 tile
    off, S_total = 32, S + 64
    if split:
        outs = tuple(torch.full((B, S_total, C), float("nan"), dtype=dtype, device="cuda") for _ in range(3))
        ref = tuple(torch.full((B, S_total, C), float("nan"), dtype=dtype, device="cuda") for _ in range(3))
        assert qkv_proj_norm_rope(xg, m, wq, wk, cos, sin, heads, out=outs, token_offset=off) is None
        qk_norm_rope(tile.clone(), wq, wk, cos, sin, heads, out=ref, token_offset=off)
        torch.cuda.synchronize()
        assert _lib.device_status() == (0, 0)
        for g, e in zip(outs, ref):
            assert torch.isnan(g[:, :off].float()).all() and torch.isnan(g[:, off + S:].float()).all()   # nothing else written
            close(g[:, off:off + S].float().cpu(), e[:, off:off + S].float().cpu(), ulps=1.0, frac=0.9995)
        got = torch.cat([t[:, off:off + S] for t in outs], dim=-1)
    else:
        got = qkv_proj_norm_rope(xg, m, wq, wk, cos, sin, heads)
        ref = qk_norm_rope(tile.clone(), wq, wk, cos, sin, heads)
        torch.cuda.synchronize()
        assert _lib.device_status() == (0, 0)
        close(got.float().cpu(), ref.float().cpu(), ulps=1.0, frac=0.9995)
    exp = R.ref_qk_norm_rope(tile.cpu().view(B * S, 3 * C), wq.cpu(), wk.cpu(), cos.cpu(), sin.cpu(), heads)
    close(got.float().cpu().view(B * S, 3 * C), exp.float(), ulps=1.0, frac=0.999)


@pytest.mark.parametrize("B,S,C,with_z,with_gate", [(2, 70, 256, False, True), (3, 50, 2240, True, True), (1, 333, 3072, False, False)])
def test_gate_residual_matches_torch(B, S, C, with_z, with_gate):
    from nunchaku_b200.ops import gate_residual

    g = torch.Generator().manual_seed(C + S)
    x, y, z = (torch.randn(B, S, C, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    mod = torch.randn(B, 6 * C, generator=g).to(torch.bfloat16).cuda()
    gate = mod.chunk(6, dim=-1)[2] if with_gate else None          # a strided view, as the blocks pass it
    got = gate_residual(x, gate, y, z if with_z else None)
    gf = gate.float().unsqueeze(1) if with_gate else 1.0
    exp = x.float() + gf * (y.float() + (z.float() if with_z else 0.0))
    assert _lib.device_status() == (0, 0)
    _bf16_close(got.float().cpu(), exp.cpu(), ulps=0.51, frac=1.0)     # fp32 arithmetic, one rounding
    # in place on x
    x2 = x.clone()
    assert gate_residual(x2, gate, y, z if with_z else None, out=x2) is x2 and torch.equal(x2, got)


def test_rowwise_kernels_in_fp16():
    """The same kernels compiled for fp16 tensors (`dtype` of their argument structs) against the same restatements."""
    from nunchaku_b200.ops import gate_residual, layernorm_modulate, linearattn_vk_mul_q, litela_attention, qk_norm_rope

    g = torch.Generator().manual_seed(77)
    B, S, heads = 2, 100, 3
    dim = heads * 128
    qkv = (torch.randn(B * S, 3 * dim, generator=g) * 2).half()
    wq, wk = (1 + 0.2 * torch.randn(128, generator=g)).half(), (1 + 0.2 * torch.randn(128, generator=g)).half()
    ang = torch.rand(S, 64, generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    exp = R.ref_qk_norm_rope(qkv, wq, wk, cos, sin, heads)
    got = qk_norm_rope(qkv.cuda().view(B, S, 3 * dim), wq.cuda(), wk.cuda(), cos.cuda(), sin.cuda(), heads).cpu().view(B * S, 3 * dim)
    assert got.dtype == torch.float16 and torch.equal(got[:, 2 * dim:], qkv[:, 2 * dim:])
    _f16_close(got[:, :2 * dim], exp[:, :2 * dim])
    # token-major split outputs
    outs = tuple(torch.zeros(B, S + 28, dim, dtype=torch.float16, device="cuda") for _ in range(3))
    qk_norm_rope(qkv.cuda().view(B, S, 3 * dim), wq.cuda(), wk.cuda(), cos.cuda(), sin.cuda(), heads, out=outs, token_offset=28)
    for i in range(3):
        assert torch.equal(outs[i][:, 28:].cpu().reshape(B * S, dim), got[:, i * dim:(i + 1) * dim])
        assert (outs[i][:, :28] == 0).all()

    x = torch.randn(B, S, 1024, generator=g).half()
    sc, sh = (torch.randn(B, 1024, generator=g) * 0.1).half(), (torch.randn(B, 1024, generator=g) * 0.1).half()
    _f16_close(layernorm_modulate(x.cuda(), sc.cuda(), sh.cuda()).cpu(), R.ref_layernorm_modulate(x, sc, sh))
    y, z = torch.randn(B, S, 1024, generator=g).half(), torch.randn(B, S, 1024, generator=g).half()
    exp = (x.double() + sc.double()[:, None, :] * (y.double() + z.double())).half()
    # one fused multiply-add in fp32, then one rounding to fp16: a double rounding against the float64 value now and then
    _f16_close(gate_residual(x.cuda(), sc.cuda(), y.cuda(), z.cuda()).cpu(), exp, ulps=1.0, frac=0.9995)
    assert torch.equal(gate_residual(x.cuda(), None, y.cuda()).cpu(), (x.float() + y.float()).half())

    lh = 5
    q3 = torch.randn(B, 700, 3 * lh * 32, generator=g).half()
    q3[..., lh * 32:] *= 6      # vk far outside fp16's precision sweet spot: sums of ~700 products of size ~20
    exp, exp_vk = R.ref_litela(q3, lh)
    got, vk = litela_attention(q3.cuda(), lh, return_vk=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert got.dtype == torch.float16 and R.rel_l2(vk.cpu(), exp_vk) <= 1e-5
    g32, e32 = got.float().cpu(), exp.float()
    assert R.rel_l2(g32, e32) <= 4e-4
    assert ((g32 - e32).abs() <= 2.0 ** -10 * e32.abs() + 1e-6).all()
    # the second half on its own (vk_mul_q_kernel): relu(Q) in place
    rq = q3[..., :lh * 32].clamp_min(0).contiguous().cuda()
    assert torch.equal(linearattn_vk_mul_q(rq, vk), got)


def test_rowwise_kernels_reject_mixed_dtypes():
    from nunchaku_b200.ops import gate_residual, qk_norm_rope

    x = torch.zeros(1, 8, 256, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        gate_residual(x, None, x.bfloat16())
    qkv = torch.zeros(1, 8, 384, dtype=torch.float16, device="cuda")
    w = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    t = torch.zeros(8, 64, device="cuda")
    with pytest.raises(ValueError):
        qk_norm_rope(qkv, w, w, t, t, 1)
