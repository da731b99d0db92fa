"""The INT4 weight quantiser (svdq_quantize_w4a4_wgt) against the CPU restatement of the reference's kernel (bf16, bit for bit)
and, when it has been built, against that kernel itself (bf16 and fp16, bit for bit), then through the GEMM."""
import pytest
import torch

import helpers as H
import ref_int4 as REF
from oracle import layouts as L
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


def _weight(N, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    w[:, ::97] *= 30                      # a few large columns: groups with very different maxima
    w[5, 64:128] = 0                      # an all-zero group (scale 0, codes 0 through 7 / 0 = inf, inf * 0 = NaN)
    w[7, :64] = 2.0 ** -100               # a tiny group (zero in fp16)
    w[9, 0] = 3.0e38 if dtype == torch.bfloat16 else 6.0e4   # and one at the top of it
    return w.to(dtype)


@pytest.mark.parametrize("N,K", [(128, 64), (256, 320), (1152, 3072)])
def test_quantize_wgt_matches_the_restatement(N, K):
    from nunchaku_b200.ops import svdq_quantize_w4a4_wgt

    w = _weight(N, K, torch.bfloat16, N + K)
    q, s = svdq_quantize_w4a4_wgt(w.cuda())
    codes, scales = R.ref_quantize_wgt_int4(w)
    assert torch.equal(L.ref_unpack_wgt_codes(q.cpu().view(torch.uint8), K), codes)
    assert torch.equal(L.ref_unpack_wscales(s.cpu()).view(torch.int16), scales.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quantize_wgt_matches_the_reference_kernel(dtype):
    from nunchaku_b200.ops import svdq_quantize_w4a4_wgt

    if not REF.has_quantize_wgt():
        pytest.skip("oracle/_ref (the reference's kernels with the weight-quantiser door) has not been built")
    w = _weight(512, 1024, dtype, 3).cuda()
    q, s = svdq_quantize_w4a4_wgt(w)
    rq, rs = REF.quantize_wgt(w)
    torch.cuda.synchronize()
    assert torch.equal(q, rq)
    assert torch.equal(s.view(torch.int16), rs.view(torch.int16))


def test_quantized_weight_runs_through_the_gemm():
    """weights quantised by the kernel, activations by the activation quantiser: the INT4 GEMM gives x w^T to 4-bit accuracy"""
    from nunchaku_b200.models.linear import SVDQW4A4Linear
    from nunchaku_b200.ops import svdq_quantize_w4a4_wgt

    N, K, M = 256, 512, 192
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    m = SVDQW4A4Linear(K, N, rank=16, bias=False, precision="int4", torch_dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        q, s = svdq_quantize_w4a4_wgt(w.cuda())
        m.qweight.copy_(q)
        m.wscales.copy_(s)
        m.smooth_factor.fill_(1.0)
        m.proj_down.zero_()
        m.proj_up.zero_()
        y = m(x.cuda().view(1, M, K)).float().cpu().view(M, N)
    ref = x.float() @ w.float().t()
    assert R.rel_l2(y, ref) <= 0.2          # two 4-bit roundings: ~0.1 each
    assert R.rel_l2(y, ref) >= 1e-3         # ... and it did go through them


def test_quantize_wgt_rejects_bad_shapes():
    from nunchaku_b200.ops import svdq_quantize_w4a4_wgt

    with pytest.raises(ValueError):
        svdq_quantize_w4a4_wgt(torch.zeros(100, 64, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        svdq_quantize_w4a4_wgt(torch.zeros(128, 64, dtype=torch.float32, device="cuda"))
