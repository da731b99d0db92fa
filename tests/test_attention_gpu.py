"""The tcgen05 attention kernel against the CPU restatement of the reference's attention (oracle.svdq_ref.ref_attention).

Floating point: the tolerance is a relative L2 error of 3e-3 for bf16 and 4e-4 for fp16, against the restatement that rounds
the probabilities to the 16-bit type as the reference does and against exact softmax attention alike.  The measured error is
2.1e-3 - 2.4e-3 / 2.9e-4, almost all of it the one rounding of the output to the 16-bit type (torch's library attention
shows the same figures on the same inputs); where the block-wise running maximum puts the rounding of the probabilities
moves it in the fourth digit."""
import pytest
import torch

from nunchaku_b200 import _lib
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu

TOL = {torch.bfloat16: (3e-3, 3e-3), torch.float16: (4e-4, 4e-4)}


def _inputs(B, H, Tq, Tk, dtype, seed, token_major=True, qmul=1.0):
    g = torch.Generator().manual_seed(seed)

    def mk(T, mul=1.0):
        if token_major:   # [B, T, H, 128] in memory, viewed [B, H, T, 128]
            return (torch.randn(B, T, H, 128, generator=g) * mul).to(dtype).transpose(1, 2)
        return (torch.randn(B, H, T, 128, generator=g) * mul).to(dtype)

    return mk(Tq, qmul), mk(Tk), mk(Tk)


def _check(q, k, v, scale=128 ** -0.5, out=None):
    from nunchaku_b200.ops import attention

    got = attention(q.cuda(), k.cuda(), v.cuda(), out=out, scale=scale)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    got = got.cpu()
    tol_p, tol_exact = TOL[q.dtype]
    assert R.rel_l2(got, R.ref_attention(q, k, v, scale)) <= tol_p
    assert R.rel_l2(got, R.ref_attention(q, k, v, scale, round_p=False)) <= tol_exact
    return got


@pytest.mark.parametrize("B,H,Tq,Tk", [(1, 1, 128, 128), (1, 2, 256, 256), (2, 3, 300, 333), (1, 2, 100, 100), (1, 1, 520, 1),
                                       (2, 2, 257, 1153)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attention_matches_oracle(B, H, Tq, Tk, dtype):
    """exact tiles, ragged query and key counts (rows past q_len unwritten, keys past kv_len masked), one key, many blocks"""
    _check(*_inputs(B, H, Tq, Tk, dtype, seed=B * 100 + Tq + Tk))


def test_attention_head_major_inputs_as_the_reference_packs_them():
    """attention_fp16's layout: q, k, v packed [B, H, T, 128], o [B, Tq, H*128], written in place"""
    from nunchaku_b200._C import ops

    q, k, v = _inputs(2, 3, 256, 384, torch.bfloat16, seed=5, token_major=False)
    o = torch.full((2, 256, 3 * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.attention_fp16(q.cuda(), k.cuda(), v.cuda(), o, 128 ** -0.5) is None
    torch.cuda.synchronize()
    assert R.rel_l2(o.cpu(), R.ref_attention(q, k, v, 128 ** -0.5)) <= TOL[torch.bfloat16][0]


def test_attention_growing_maximum_rescales_the_accumulator():
    """keys sorted so that every block raises the row maximum by far more than the rescale threshold"""
    B, H, T = 1, 2, 1024
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, H, 256, 128, generator=g).abs().to(torch.bfloat16)
    k = (torch.randn(B, H, T, 128, generator=g).abs() * torch.linspace(0.05, 3.0, T)[None, None, :, None]).to(torch.bfloat16)
    v = torch.randn(B, H, T, 128, generator=g).to(torch.bfloat16)
    _check(q, k, v)


def test_attention_strided_output_and_rows_past_q_len_untouched():
    q, k, v = _inputs(1, 2, 200, 300, torch.bfloat16, seed=3)
    buf = torch.full((1, 256, 2 * 128 + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    out = buf[:, :200, :256]
    _check(q, k, v, out=out)
    assert (buf[:, 200:] == 7).all() and (buf[:, :, 256:] == 7).all()


def test_attention_constant_values_give_that_constant():
    """size-independent property at the FLUX sequence length: softmax rows sum to one"""
    B, H, T = 1, 2, 4608
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, T, H, 128, device="cuda", generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(B, T, H, 128, device="cuda", generator=g).bfloat16().transpose(1, 2)
    v = torch.full((B, T, H, 128), 0.75, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    from nunchaku_b200.ops import attention

    o = attention(q, k, v)
    assert (o.float() - 0.75).abs().max().item() <= 0.75 * 2 ** -7   # the probabilities are rounded to bf16 (2^-9 each, averaged)


def test_attention_flux_size_against_fp32_softmax_on_the_gpu():
    """[1, 24, 4608, 128]: fp32 softmax attention computed with torch on the GPU, per head"""
    from nunchaku_b200.ops import attention

    B, H, T = 1, 24, 4608
    g = torch.Generator(device="cuda").manual_seed(2)
    q, k, v = (torch.randn(B, T, H, 128, device="cuda", generator=g).bfloat16().transpose(1, 2) for _ in range(3))
    o = attention(q, k, v).view(B, T, H, 128)
    for h in range(0, H, 5):
        s = (q[0, h].float() @ k[0, h].float().T) * 128 ** -0.5
        r = torch.softmax(s, dim=-1) @ v[0, h].float()
        assert R.rel_l2(o[0, :, h].float().cpu(), r.cpu()) <= 3e-3


def test_attention_rejects_what_it_cannot_run():
    from nunchaku_b200.ops import attention

    q = torch.zeros(1, 2, 64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        attention(q, q, q)
    q = torch.zeros(1, 2, 64, 128, dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        attention(q, q, q)


def test_attention_degenerate_inputs():
    """one query; all-equal scores (uniform weights: the mean of V); a scale so large that the softmax is one-hot; magnitudes
    near the top of bf16's range of useful scores (products of ~1e4 before scaling)"""
    from nunchaku_b200.ops import attention

    g = torch.Generator().manual_seed(17)
    q, k, v = _inputs(1, 2, 1, 300, torch.bfloat16, seed=1)
    o1 = attention(q.cuda(), k.cuda(), v.cuda()).float().cpu()
    e1 = R.ref_attention(q, k, v, 128 ** -0.5, round_p=False).float()
    assert R.rel_l2(o1, e1) <= 5e-3 and (o1 - e1).abs().max() <= 2.0 ** -8    # 256 values only: a looser norm, plus an absolute bound
    q, k, v = _inputs(1, 2, 130, 260, torch.bfloat16, seed=2)
    o = attention(torch.zeros_like(q).cuda(), k.cuda(), v.cuda()).float().cpu()
    mean_v = v.float().mean(dim=2).reshape(1, 1, 2 * 128).expand(1, 130, 256)
    assert R.rel_l2(o, mean_v) <= 3e-3
    # one-hot: out = V[argmax]
    o = attention(q.cuda(), k.cuda(), v.cuda(), scale=50.0).cpu()
    s = q.float() @ k.float().transpose(-1, -2)
    top2 = s.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) * 50.0 * 1.4427 > 30      # rows whose runner-up weighs less than 2^-30
    idx = s.argmax(-1)                                               # [1, 2, 130]
    exp = torch.gather(v, 2, idx[..., None].expand(1, 2, 130, 128)).transpose(1, 2).reshape(1, 130, 256)
    m = clear.transpose(1, 2).reshape(1, 130, 2, 1).expand(1, 130, 2, 128).reshape(1, 130, 256)
    assert clear.float().mean() > 0.5 and torch.equal(o[m], exp[m])
    assert torch.isfinite(o.float()).all()
    q2 = (torch.randn(1, 2, 64, 128, generator=g) * 30).to(torch.bfloat16)
    k2 = (torch.randn(1, 2, 200, 128, generator=g) * 30).to(torch.bfloat16)
    _check(q2, k2, v[:, :, :200])
