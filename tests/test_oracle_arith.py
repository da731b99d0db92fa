"""Known-answer tests pinning the oracle's own arithmetic to the rounding rules it cites
(gemm_utils.cuh:206-264, gemm_w4a4.cuh:85-187,429-523)."""
import torch

from oracle import fmt
from oracle import svdq_ref as R


def test_e2m1_round_to_nearest_even_and_saturation():
    v = torch.tensor([0.0, 0.2, 0.25, 0.26, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 5.01, 6.0, 7.0, 1e9])
    exp = [0, 0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 4, 5, 6, 6, 6, 7, 7, 7, 7]
    assert fmt.e2m1_encode(v).tolist() == exp
    assert fmt.e2m1_encode(-v[1:]).tolist() == [e | 8 for e in exp[1:]]
    assert fmt.e2m1_encode(torch.tensor([-0.0, -0.1])).tolist() == [8, 8]  # the sign of a zero result is kept
    assert torch.equal(fmt.e2m1_decode(torch.arange(16)), torch.tensor(
        [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]))


def test_e4m3_round_and_clamp():
    v = torch.tensor([0.0, 2 ** -10, 2 ** -9, 1.0, 1.0625, 1.125, 448.0, 1000.0])
    assert fmt.e4m3_encode(v).tolist() == [0, 0, 1, 0x38, 0x38, 0x39, 0x7E, 0x7E]


def test_int4_round_half_even_and_saturation():
    v = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 7.4, 7.5, 9.0, -8.5, -9.0, float("nan")])
    assert fmt.int4_decode(fmt.int4_encode(v, False), False).tolist() == [0, 2, 2, 0, -2, 7, 7, 7, -8, -8, 0]
    assert fmt.int4_decode(fmt.int4_encode(torch.tensor([15.5, 16.0, -1.0, 14.5]), True), True).tolist() == [15, 15, 0, 14]


def test_group_quantize_hand_case_nvfp4():
    # one group of 16: max 12 -> scale 2.0 exactly (12 * fp32(1/6) rounds to 2), codes = v / 2
    v = torch.zeros(1, 16, dtype=torch.bfloat16)
    v[0, :6] = torch.tensor([12.0, -6.0, 3.0, 1.0, 0.5, -0.4], dtype=torch.bfloat16)
    codes, scales, _ = R.group_quantize(v, fp4=True)
    assert scales.tolist() == [[0x40]]  # e4m3 2.0
    assert codes[0, :6].tolist() == [7, 8 | 5, 3, 1, 0, 8 | 0]   # 6, -3, 1.5, .5, .25->0 (tie to even), -.2->-0
    assert codes[0, 6:].tolist() == [0] * 10


def test_group_quantize_zero_group_and_scale_clamp():
    v = torch.zeros(2, 16, dtype=torch.bfloat16)
    v[1, 0] = 6000.0
    codes, scales, _ = R.group_quantize(v, fp4=True)
    assert scales[0, 0].item() == 0 and codes[0].sum().item() == 0
    assert scales[0, 1].item() == 0x7E          # 1000 clamps to 448
    assert codes[1, 0].item() == 7              # 6000 / 448 saturates to 6


def test_group_quantize_hand_case_int4():
    v = torch.zeros(1, 64, dtype=torch.bfloat16)
    v[0, :4] = torch.tensor([7.0, -3.5, 0.5, -7.0], dtype=torch.bfloat16)
    codes, scales, _ = R.group_quantize(v, fp4=False)
    assert scales[0, 0].item() == 1.0
    assert fmt.int4_decode(codes[0, :4], False).tolist() == [7, -4, 0, -7]  # -3.5 -> -4 and .5 -> 0: ties to even


def test_quantize_then_gemm_approximates_master():
    for fp4 in (True, False):
        x = R.make_activations(300, 512, seed=0)
        lin = R.make_linear(512, 384, 32, fp4=fp4, x_absmax=x.float().abs().amax(0), mode="svd")
        q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
        assert q.codes.shape == (512, 512) and q.lora_act.shape == (512, 32)
        assert q.codes[300:].sum() == 0  # padding rows quantise to zero codes / zero scales
        y = R.ref_gemm(q, lin, M=300)
        assert R.rel_l2(y, x.float() @ lin.master.t() + lin.bias.float()) < 0.12


def test_requantize_unsigned_shift():
    y = torch.randn(256, 128) * 0.5
    nxt = R.make_linear(128, 128, 32, fp4=False, seed=4)
    act = R.gelu_f32(y)
    q = R.ref_requantize(act, nxt, M_pad=256, unsigned=True)
    assert q.unsigned and int(q.codes.max()) <= 15
    deq = R.dequant_act(q)
    want = (act.to(torch.bfloat16).float() + R.INT4_UNSIGNED_SHIFT) / nxt.smooth.float()
    assert R.rel_l2(deq, want) < 0.08


def test_ref_litela_against_explicit_loops():
    """The vectorised linear-attention restatement equals the formula written out token by token
    (epilogues.cuh:599-656 for vk, :730-756 for the product with q and the division)."""
    import torch

    from oracle import svdq_ref as R

    g = torch.Generator().manual_seed(0)
    B, S, heads = 2, 5, 2
    D = heads * 32
    qkv = torch.randn(B, S, 3 * D, generator=g).to(torch.bfloat16)
    out, vk = R.ref_litela(qkv, heads)
    x = qkv.double()
    for b in range(B):
        for h in range(heads):
            ref_vk = torch.zeros(33, 32, dtype=torch.float64)
            for t in range(S):
                k = x[b, t, D + 64 * h: D + 64 * h + 32].clamp_min(0)
                v = x[b, t, D + 64 * h + 32: D + 64 * h + 64]
                ref_vk[:32] += v[:, None] * k[None, :]
                ref_vk[32] += k
            assert torch.allclose(vk[b, h].double(), ref_vk, rtol=1e-6, atol=1e-6)
            for t in range(S):
                q = x[b, t, 32 * h: 32 * h + 32].clamp_min(0)
                o = ref_vk.float().double() @ q
                exp = (o[:32].float() / (o[32].float() + 1e-6)).to(torch.bfloat16)
                assert torch.equal(out[b, t, 32 * h: 32 * h + 32], exp)


def test_group_quantize_flags_rounding_ties():
    """An exact tie (7 * v / max = k + 0.5) is flagged: there the reference's approximate reciprocal decides the code."""
    v = torch.zeros(1, 64)
    v[0, 0] = 14.0            # group maximum: scale = 2
    v[0, 1] = 3.0             # 3 / 2 = 1.5: a tie
    v[0, 2] = 3.25            # 1.625: not a tie
    codes, scales, tie = R.group_quantize(v.to(torch.bfloat16), fp4=False)
    assert bool(tie[0, 1]) and not bool(tie[0, 2]) and not bool(tie[0, 0])
    v = torch.zeros(1, 16)
    v[0, 0] = 6.0             # scale = 1
    v[0, 1] = 2.5             # midway between 2 and 3
    v[0, 2] = 2.75
    codes, scales, tie = R.group_quantize(v.to(torch.bfloat16), fp4=True)
    assert bool(tie[0, 1]) and not bool(tie[0, 2])


def test_ref_attention_is_softmax_attention():
    """The attention restatement against plain loops over rows (exact softmax in float64), and its one deliberate deviation:
    probabilities rounded to the 16-bit type before the product with v (attention.cuh packs P as 16-bit fragments)."""
    g = torch.Generator().manual_seed(4)
    B, H, Tq, Tk = 1, 2, 5, 37
    q = torch.randn(B, H, Tq, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, Tk, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, Tk, 128, generator=g).to(torch.bfloat16)
    scale = 128 ** -0.5
    exact = R.ref_attention(q, k, v, scale, round_p=False)
    rounded = R.ref_attention(q, k, v, scale)
    for h in range(H):
        for t in range(Tq):
            s = (k[0, h].double() @ q[0, h, t].double()) * scale
            p = torch.exp(s - s.max())
            o = (p[:, None] * v[0, h].double()).sum(0) / p.sum()
            assert torch.allclose(exact[0, t, 128 * h: 128 * h + 128].double(), o, rtol=2 ** -8, atol=1e-6)
    assert R.rel_l2(rounded, exact) < 3e-3
    assert R.ref_attention(q.half(), k.half(), v.half(), scale).dtype == torch.float16


def test_ref_quantize_wgt_int4_by_hand():
    """The weight-quantiser restatement on hand-computed groups: every step in bf16 (gemm_w4a4.cuh:527-620)."""
    w = torch.zeros(1, 128, dtype=torch.bfloat16)
    w[0, 0], w[0, 1], w[0, 2], w[0, 3] = 7.0, -7.0, 3.5, 0.49       # max 7: scale 1, rscale 1
    w[0, 64], w[0, 65] = 1.0, -1.0                                   # max 1: scale bf16(1/7), rscale 7
    codes, scales = R.ref_quantize_wgt_int4(w)
    assert codes[0, :4].tolist() == [7, 9, 4, 0]                     # 7, -7 (two's complement nibble), rint(3.5) = 4 (even), 0
    assert codes[0, 64:66].tolist() == [7, 9]
    assert scales[0, 0].item() == 1.0 and scales[1, 0] == torch.tensor(1.0 / 7.0).to(torch.bfloat16)
    assert (codes[0, 4:64] == 0).all()
    z, zs = R.ref_quantize_wgt_int4(torch.zeros(1, 64, dtype=torch.bfloat16))
    assert (z == 0).all() and zs[0, 0].item() == 0.0                 # inf * 0 = NaN -> 0
