"""Parity of the CUDA W4A4 GEMM (through the C ABI) with the CPU oracle.

Tolerance: the path's specification is relative L2 <= 1e-2 against the
dequantise-then-matmul fp32 reference; the bf16 rounding of the output alone is ~1.7e-3,
so the tests hold the kernel to 4e-3."""
import pytest
import torch

import helpers as H
from oracle import fmt
from oracle import layouts as L
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu

REL_L2_SPEC = 1e-2
REL_L2_TIGHT = 4e-3


def gemm(q, lin, M, use_lora=True, fuse_silu=False, act_layout="native", lora_scales=None):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    sd = {k: v.cuda() for k, v in H.packed_params(lin).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, act_layout)]
    out = torch.full((M, lin.N), float("nan"), dtype=torch.bfloat16, device="cuda")
    svdq_gemm_w4a4_cuda(
        act=codes, wgt=sd["qweight"], out=out, ascales=scales, wscales=sd["wscales"],
        lora_act_in=lora if use_lora else None, lora_up=sd["proj_up"] if use_lora else None,
        bias=sd.get("bias"), fp4=lin.fp4, alpha=lin.wtscale if lin.fp4 else 1.0, wcscales=sd.get("wcscales"),
        fuse_silu=fuse_silu, lora_scales=lora_scales,
        act_layout=_lib.LAYOUT_NATIVE if act_layout == "native" else _lib.LAYOUT_REFERENCE,
    )
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    return out.float().cpu()


def problem(M, K, N, Rk, fp4, seed=0, wcscales=True, bias=True):
    x = R.make_activations(M, K, seed=seed)
    lin = R.make_linear(K, N, Rk, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=seed + 1, mode="svd",
                        wcscales=wcscales and fp4, bias=bias)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    return x, lin, q


def test_nvfp4_exact_small_integers():
    """Known answers: all codes 1.0 and power-of-two scales give exactly representable sums."""
    M, K, N = 256, 256, 384
    acodes = torch.full((M, K), 2, dtype=torch.uint8)
    wcodes = torch.full((N, K), 2, dtype=torch.uint8)
    asc = fmt.e4m3_encode((torch.arange(M) % 4 + 1).float().exp2())[None, :].expand(K // 16, M).contiguous()
    wsc = fmt.e4m3_encode((torch.arange(K // 16) % 3).float().exp2())[:, None].expand(K // 16, N).contiguous()
    q = R.QuantOut(acodes, asc, torch.zeros(M, 32), True)
    lin = R.Linear(K, N, 32, True, wcodes, wsc, torch.ones(K, dtype=torch.bfloat16), torch.zeros(32, K, dtype=torch.bfloat16),
                   torch.zeros(N, 32, dtype=torch.bfloat16), None, 1.0, torch.ones(N, dtype=torch.bfloat16))
    exp = R.ref_gemm(q, lin, M=M, use_lora=False)
    assert torch.equal(gemm(q, lin, M, use_lora=False), exp)


@pytest.mark.parametrize("M,K,N,Rk,use_lora", [
    (256, 128, 128, 32, False),
    (256, 256, 384, 32, True),
    (300, 512, 640, 32, True),      # ragged M, N not a multiple of the 256-column tile
    (1, 128, 128, 16, True),
    (256, 384, 128, 64, True),
    (512, 640, 1280, 128, True),
    (1024, 3072, 3072, 32, True),
    (300, 256, 384, 80, True),      # ranks that are not a multiple of 32, and above 128
    (256, 256, 256, 272, True),
])
def test_nvfp4_gemm_matches_oracle(M, K, N, Rk, use_lora):
    x, lin, q = problem(M, K, N, Rk, True, seed=M + N)
    exp = R.ref_gemm(q, lin, M=M, use_lora=use_lora)
    got = gemm(q, lin, M, use_lora=use_lora)
    assert not torch.isnan(got).any()
    assert R.rel_l2(got, exp) <= REL_L2_TIGHT


def test_nvfp4_gemm_silu_and_no_bias():
    x, lin, q = problem(300, 256, 384, 32, True, seed=4, bias=False)
    exp = R.ref_gemm(q, lin, M=300, act="silu")
    assert R.rel_l2(gemm(q, lin, 300, fuse_silu=True), exp) <= REL_L2_TIGHT


def test_nvfp4_gemm_lora_scales():
    x, lin, q = problem(256, 256, 256, 32, True, seed=5)
    exp = R.ref_gemm(q, lin, M=256, lora_scales=[0.5, 2.0])
    assert R.rel_l2(gemm(q, lin, 256, lora_scales=[0.5, 2.0]), exp) <= REL_L2_TIGHT


def test_nvfp4_gemm_reference_layout_inputs():
    x, lin, q = problem(300, 256, 384, 32, True, seed=6)
    exp = R.ref_gemm(q, lin, M=300)
    assert R.rel_l2(gemm(q, lin, 300, act_layout="reference"), exp) <= REL_L2_TIGHT


def test_nvfp4_gemm_rows_beyond_M_untouched():
    """`out` has the true M rows; nothing may be written past it (gemm_base.cuh:544-548)."""
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    M = 300
    x, lin, q = problem(M, 256, 384, 32, True, seed=7)
    sd = {k: v.cuda() for k, v in H.packed_params(lin).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    buf = torch.full((M + 64, lin.N), 7.0, dtype=torch.bfloat16, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd["qweight"], out=buf[:M], ascales=scales, wscales=sd["wscales"],
                        lora_act_in=lora, lora_up=sd["proj_up"], bias=sd["bias"], fp4=True, alpha=lin.wtscale,
                        wcscales=sd["wcscales"])
    torch.cuda.synchronize()
    assert (buf[M:] == 7.0).all()


def test_nvfp4_headline_config1_slice():
    """The 4608 x 3072 x 21504 NVFP4 workload (FLUX single-block fused input projection, rank 32) on all its rows."""
    M, K, N = 4608, 3072, 21504
    x, lin, q = problem(M, K, N, 32, True, seed=0, wcscales=False)
    got = gemm(q, lin, M)
    rows = torch.arange(0, M, 9)  # the oracle matmul on every 9th row keeps the CPU time in seconds
    q_rows = R.QuantOut(q.codes[rows], q.scales[:, rows].contiguous(), q.lora_act[rows], True)
    exp = R.ref_gemm(q_rows, lin)
    assert R.rel_l2(got[rows], exp) <= REL_L2_TIGHT
    # size-independent property: linearity in the low-rank input (epilogue is affine in lora_act)
    q2 = R.QuantOut(q.codes, q.scales, q.lora_act * 2.0, True)
    got2 = gemm(q2, lin, M)
    lora_term = (q.lora_act[rows] @ lin.lora_up.float().t())
    assert R.rel_l2((got2 - got)[rows], lora_term) <= 2e-2  # difference of two bf16-rounded outputs


def test_linear_module_end_to_end():
    """SVDQW4A4Linear.forward = quantise -> GEMM, against the oracle and the bf16 master weight."""
    M, K, N = 600, 512, 768
    x = R.make_activations(M, K, seed=1)
    lin = R.make_linear(K, N, 32, fp4=True, x_absmax=x.float().abs().amax(0), seed=2, mode="svd")
    m = H.to_module(lin)
    y = m(x.cuda().view(2, M // 2, K)).float().cpu().view(M, N)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=True)
    # the quantiser's codes equal the oracle's except on rounding ties (either neighbour is right there), so the GEMM is
    # checked on the codes the GPU produced, and the whole chain against the oracle chain within the path's tolerance
    gq = H.module_quantize(m, x.cuda())
    H.assert_codes_match(gq.codes, q, rows=slice(0, M))
    assert R.rel_l2(y, R.ref_gemm(gq, lin, M=M)) <= REL_L2_TIGHT
    assert R.rel_l2(y, R.ref_gemm(q, lin, M=M)) <= REL_L2_SPEC
    assert R.rel_l2(y, x.float() @ lin.master.t() + lin.bias.float()) <= 0.12  # 4-bit quantisation error


# ----------------------------------------------------------------------------- INT4 (group 64)
@pytest.mark.parametrize("M,K,N,Rk,use_lora", [
    (256, 128, 128, 32, False),
    (256, 256, 384, 32, True),
    (300, 512, 640, 16, True),
    (1, 128, 256, 32, True),
    (512, 640, 1280, 64, True),
])
def test_int4_gemm_matches_oracle(M, K, N, Rk, use_lora):
    x, lin, q = problem(M, K, N, Rk, False, seed=M + N)
    exp = R.ref_gemm(q, lin, M=M, use_lora=use_lora)
    got = gemm(q, lin, M, use_lora=use_lora)
    assert not torch.isnan(got).any()
    assert R.rel_l2(got, exp) <= REL_L2_TIGHT


def test_int4_exact_small_integers():
    """All codes +-1..7 with unit scales: the int32 group sums and their fp32 total are exact."""
    M, K, N = 256, 256, 256
    g = torch.Generator().manual_seed(3)
    acodes = torch.randint(0, 16, (M, K), generator=g, dtype=torch.uint8)
    wcodes = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    ones_a = torch.ones(K // 64, M, dtype=torch.bfloat16)
    ones_w = torch.ones(K // 64, N, dtype=torch.bfloat16)
    q = R.QuantOut(acodes, ones_a, torch.zeros(M, 32), False)
    lin = R.Linear(K, N, 32, False, wcodes, ones_w, torch.ones(K, dtype=torch.bfloat16), torch.zeros(32, K, dtype=torch.bfloat16),
                   torch.zeros(N, 32, dtype=torch.bfloat16), None)
    exp = R.ref_gemm(q, lin, M=M, use_lora=False)          # |sum| <= 256*64 = 16384: needs 15 bits, bf16 has 8
    got = gemm(q, lin, M, use_lora=False)
    assert torch.equal(got, exp.to(torch.bfloat16).float())


@pytest.mark.parametrize("unsigned", [False, True])
def test_int4_scale_range_edges(unsigned):
    """Rows whose group scales span far more than fp16's exponent range: huge rows (scales far above 4094), tiny rows
    (1e-6: code * scale would be an fp16 subnormal), and u4 codes 9 / 11 / 13 / 15 against scales with a full bf16 mantissa.
    The reference multiplies integer sums by bf16 scales and has no such limits; here a power of two is taken out of each
    row before the fp16 conversion.  Every ROW must match the oracle (a global norm would hide the small rows):
    relative L2 per row <= 6e-3 (bf16 output rounding is 2e-3 of an element)."""
    M, K, N = 256, 512, 256
    g = torch.Generator().manual_seed(17)
    lin = R.make_linear(K, N, 32, fp4=False, seed=19, bias=False)
    codes = torch.randint(0, 16, (M, K), generator=g, dtype=torch.uint8)
    if unsigned:
        codes[1::2] = torch.tensor([9, 11, 13, 15], dtype=torch.uint8)[torch.randint(0, 4, (M // 2, K), generator=g)]
    expo = (torch.arange(M) % 61 - 30).float()                      # row magnitudes 2^-30 .. 2^30
    mant = 1.0 + torch.randint(0, 128, (K // 64, M), generator=g).float() / 128.0     # full 8-bit mantissas
    within = torch.randint(-6, 1, (K // 64, M), generator=g).float()                  # groups up to 64x below the row's largest
    scales = (mant * torch.exp2(expo[None, :] + within)).to(torch.bfloat16)
    scales[:, 5] = 0                                                 # an all-zero row
    scales[0, 7] = 0                                                 # a zero group
    lora = torch.randn(M, 32, generator=g) * torch.exp2(expo)[:, None] * 4.0
    lora[5] = 0
    q = R.QuantOut(codes, scales, lora, False, unsigned)
    exp = R.ref_gemm(q, lin, M=M)
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda
    sd = {k: v.cuda() for k, v in H.packed_params(lin).items()}
    c, s_, la = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    svdq_gemm_w4a4_cuda(act=c, wgt=sd["qweight"], out=out, ascales=s_, wscales=sd["wscales"], lora_act_in=la, lora_up=sd["proj_up"],
                        fp4=False, act_unsigned=unsigned, act_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    assert not got[5].any()
    rows = torch.arange(M) != 5
    err = (got - exp)[rows].norm(dim=1) / exp[rows].norm(dim=1)
    assert err.max().item() <= 6e-3, f"worst row {int(err.argmax())}: {err.max().item():.3e}"


def test_int4_gemm_unsigned_activations_and_silu():
    """u4 activation codes (the post-GELU shifted path of the reference, act_unsigned=True)."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    M, K, N = 300, 256, 384
    lin = R.make_linear(K, N, 32, fp4=False, seed=8)
    y = torch.rand(M, K) * 2.0          # non-negative "activated" values
    q = R.ref_requantize(y, lin, M_pad=512, unsigned=True)
    exp = R.ref_gemm(q, lin, M=M, act="silu")
    sd = {k: v.cuda() for k, v in H.packed_params(lin).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd["qweight"], out=out, ascales=scales, wscales=sd["wscales"], lora_act_in=lora,
                        lora_up=sd["proj_up"], bias=sd["bias"], fp4=False, act_unsigned=True, fuse_silu=True,
                        act_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert R.rel_l2(out.float().cpu(), exp) <= REL_L2_TIGHT


def test_int4_headline_config0():
    """The INT4 group-64 workload M=4096, K=3072, N=3072, rank 32, through the module."""
    M, K, N = 4096, 3072, 3072
    x = R.make_activations(M, K, seed=0)
    lin = R.make_linear(K, N, 32, fp4=False, x_absmax=x.float().abs().amax(0), seed=0, mode="literal")
    m = H.to_module(lin)
    y = m(x.cuda().view(1, M, K)).float().cpu().view(M, N)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    gq = H.module_quantize(m, x.cuda())       # the GPU quantiser's own codes (equal to the oracle's except on rounding ties)
    H.assert_codes_match(gq.codes, q, rows=slice(0, M))
    rows = torch.arange(0, M, 8)
    g_rows = R.QuantOut(gq.codes[rows], gq.scales[:, rows].contiguous(), gq.lora_act[rows], False)
    assert R.rel_l2(y[rows], R.ref_gemm(g_rows, lin)) <= REL_L2_TIGHT
    q_rows = R.QuantOut(q.codes[rows], q.scales[:, rows].contiguous(), q.lora_act[rows], False)
    assert R.rel_l2(y[rows], R.ref_gemm(q_rows, lin)) <= REL_L2_SPEC


# ----------------------------------------------------------------------------- fused GELU + next-layer requantisation
def _requant_case(M, K, N, R1, R2, seed, with_out=True):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    x = R.make_activations(M, K, seed=seed)
    fc1 = R.make_linear(K, N, R1, fp4=True, x_absmax=x.float().abs().amax(0), seed=seed + 1, mode="svd", wcscales=True)
    fc2 = R.make_linear(N, 256, R2, fp4=True, x_absmax=torch.rand(N) + 0.5, seed=seed + 2)
    q = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=True)
    M_pad = q.codes.shape[0]
    sd1 = {k: v.cuda() for k, v in H.packed_params(fc1).items()}
    sd2 = {k: v.cuda() for k, v in H.packed_params(fc2).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") if with_out else None
    qout = torch.zeros(M_pad, N // 2, dtype=torch.uint8, device="cuda")
    osc = torch.zeros(N // 16, M_pad, dtype=torch.float8_e4m3fn, device="cuda")
    la2 = torch.full((M_pad, R2), float("nan"), dtype=torch.float32, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd1["qweight"], out=out, qout=qout, ascales=scales, wscales=sd1["wscales"], oscales=osc,
                        lora_act_in=lora, lora_up=sd1["proj_up"], lora_down=sd2["proj_down"], lora_act_out=la2,
                        bias=sd1["bias"], smooth_factor=sd2["smooth_factor"], fp4=True, alpha=fc1.wtscale,
                        wcscales=sd1["wcscales"], act_layout=_lib.LAYOUT_NATIVE, out_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    got = H.unpack_quant_out(qout, osc, la2, N, True, "native")
    return x, fc1, fc2, q, out, got, M_pad


@pytest.mark.parametrize("M,K,N,R1,R2", [(256, 256, 384, 32, 32), (300, 512, 640, 32, 16), (1024, 1024, 3072, 32, 32), (256, 128, 256, 16, 64),
                                         (300, 256, 384, 32, 48), (256, 256, 640, 32, 128), (256, 128, 256, 16, 208)])
def test_nvfp4_gemm_gelu_requant(M, K, N, R1, R2):
    x, fc1, fc2, q, out, got, M_pad = _requant_case(M, K, N, R1, R2, seed=M + N)
    # (1) the bf16 activated output matches the oracle
    y = R.ref_gemm(q, fc1, M=M, act="gelu")
    assert R.rel_l2(out.float().cpu(), y) <= REL_L2_TIGHT
    # (2) given the kernel's own bf16 output, its codes / scales are bit-exact and its LoRA-down tight
    exp = R.ref_requantize(out.float().cpu(), fc2, M_pad=M_pad, unsigned=False)
    H.assert_codes_match(got.codes, exp, rows=slice(0, M), what="requantised codes (given the kernel's own output)")
    assert torch.equal(got.scales[:, :M], exp.scales[:, :M])
    err = (got.lora_act[:M] - exp.lora_act[:M]).abs().max().item()
    assert err <= 2e-5 * max(exp.lora_act.abs().max().item(), 1.0) + 1e-6
    # (3) against the fp32 oracle chain: dequantised values within the GEMM tolerance of the 4-bit grid
    exp2 = R.ref_requantize(y, fc2, M_pad=M_pad, unsigned=False)
    assert R.rel_l2(R.dequant_act(got)[:M], R.dequant_act(exp2)[:M]) <= 2e-2


@pytest.mark.parametrize("R2", [32, 96])     # 96: the ranks above 64 come from a bf16 copy of the output in the workspace
def test_nvfp4_gemm_requant_without_out_and_padding_rows(R2):
    x, fc1, fc2, q, out, got, M_pad = _requant_case(300, 256, 384, 32, R2, seed=3, with_out=False)
    y = R.ref_gemm(q, fc1, act="gelu")                     # all M_pad rows: padding rows are bias-only
    exp = R.ref_requantize(y, fc2, M_pad=M_pad, unsigned=False)
    assert R.rel_l2(R.dequant_act(got), R.dequant_act(exp)) <= 2e-2
    assert R.rel_l2(got.lora_act, exp.lora_act) <= 1e-2


def test_fused_gelu_mlp_matches_oracle_chain():
    """nunchaku_b200.ops.fused_gelu_mlp (fc1 -> GELU -> requant -> fc2) vs the oracle, the FLUX MLP geometry scaled down."""
    from nunchaku_b200.ops import fused_gelu_mlp

    M, K, N1 = 600, 512, 2048
    x = R.make_activations(M, K, seed=5)
    fc1 = R.make_linear(K, N1, 32, fp4=True, x_absmax=x.float().abs().amax(0), seed=6, mode="svd")
    q1 = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=True)
    h = R.ref_gemm(q1, fc1, M=M, act="gelu")
    fc2 = R.make_linear(N1, K, 32, fp4=True, x_absmax=h.abs().amax(0).clamp(min=1e-3), seed=7, mode="svd")
    q2 = R.ref_requantize(h, fc2, M_pad=q1.codes.shape[0], unsigned=False)
    y = R.ref_gemm(q2, fc2, M=M)
    m1, m2 = H.to_module(fc1), H.to_module(fc2)
    got = fused_gelu_mlp(x.cuda().view(1, M, K), m1, m2).float().cpu().view(M, K)
    assert R.rel_l2(got, y) <= 2e-2
    # and against the bf16 master weights: 4-bit quantisation error of two stacked layers
    ref = torch.nn.functional.gelu(x.float() @ fc1.master.t() + fc1.bias.float(), approximate="tanh") @ fc2.master.t() + fc2.bias.float()
    assert R.rel_l2(got, ref) <= 0.2


def _int4_requant_case(M, K, N, R1, R2, seed, with_out=True):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    x = R.make_activations(M, K, seed=seed)
    fc1 = R.make_linear(K, N, R1, fp4=False, x_absmax=x.float().abs().amax(0), seed=seed + 1, mode="svd")
    fc2 = R.make_linear(N, 256, R2, fp4=False, x_absmax=torch.rand(N) + 0.5, seed=seed + 2)
    q = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=False)
    M_pad = q.codes.shape[0]
    sd1 = {k: v.cuda() for k, v in H.packed_params(fc1).items()}
    sd2 = {k: v.cuda() for k, v in H.packed_params(fc2).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") if with_out else None
    qout = torch.zeros(M_pad, N // 2, dtype=torch.uint8, device="cuda")
    osc = torch.zeros(N // 64, M_pad, dtype=torch.bfloat16, device="cuda")
    la2 = torch.full((M_pad, R2), float("nan"), dtype=torch.float32, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd1["qweight"], out=out, qout=qout, ascales=scales, wscales=sd1["wscales"], oscales=osc,
                        lora_act_in=lora, lora_up=sd1["proj_up"], lora_down=sd2["proj_down"], lora_act_out=la2,
                        bias=sd1["bias"], smooth_factor=sd2["smooth_factor"], fp4=False,
                        act_layout=_lib.LAYOUT_NATIVE, out_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    got = H.unpack_quant_out(qout, osc, la2, N, False, "native")
    got.unsigned = True
    return x, fc1, fc2, q, out, got, M_pad


@pytest.mark.parametrize("M,K,N,R1,R2", [(256, 256, 384, 32, 32), (300, 512, 640, 32, 16), (1024, 1024, 3072, 32, 32), (256, 128, 256, 16, 64),
                                         (300, 256, 384, 32, 96), (256, 128, 256, 160, 144)])
def test_int4_gemm_gelu_requant(M, K, N, R1, R2):
    """INT4 chain of the reference (gemm_w4a4_launch_impl.cuh:282-309): GELU, LoRA-down of the next layer on the activated
    value, then u4 codes of (y + 0.171875) / smooth with bf16 group-64 scales."""
    x, fc1, fc2, q, out, got, M_pad = _int4_requant_case(M, K, N, R1, R2, seed=M + N)
    y = R.ref_gemm(q, fc1, M=M, act="gelu")
    assert R.rel_l2(out.float().cpu(), y) <= REL_L2_TIGHT
    # given the kernel's own bf16 output, its codes / scales are bit-exact and its LoRA-down tight
    exp = R.ref_requantize(out.float().cpu(), fc2, M_pad=M_pad, unsigned=True)
    H.assert_codes_match(got.codes, exp, rows=slice(0, M), what="requantised codes (given the kernel's own output)")
    assert torch.equal(got.scales[:, :M].view(torch.int16), exp.scales[:, :M].view(torch.int16))
    err = (got.lora_act[:M] - exp.lora_act[:M]).abs().max().item()
    assert err <= 2e-5 * max(exp.lora_act.abs().max().item(), 1.0) + 1e-6
    # against the fp32 oracle chain: dequantised values within the GEMM tolerance of the 4-bit grid
    exp2 = R.ref_requantize(y, fc2, M_pad=M_pad, unsigned=True)
    assert R.rel_l2(R.dequant_act(got)[:M], R.dequant_act(exp2)[:M]) <= 2e-2


def test_int4_gemm_requant_without_out_is_deterministic():
    torch.manual_seed(0)   # the next layer's smoothing factors come from the global generator
    a = _int4_requant_case(300, 256, 384, 32, 32, seed=3, with_out=False)[5]
    torch.manual_seed(0)
    b = _int4_requant_case(300, 256, 384, 32, 32, seed=3, with_out=False)[5]
    assert torch.equal(a.codes, b.codes) and torch.equal(a.lora_act, b.lora_act)
    assert torch.equal(a.scales.view(torch.int16), b.scales.view(torch.int16))


def test_fused_gelu_mlp_int4_matches_oracle_chain():
    """fused_gelu_mlp on an INT4 pair of layers: fc2 consumes the shifted u4 codes (act_unsigned); the oracle chain
    does the same, so the +0.171875 shift appears on both sides (the reference folds its compensation into fc2's
    bias offline)."""
    from nunchaku_b200.ops import fused_gelu_mlp

    M, K, N1 = 600, 512, 2048
    x = R.make_activations(M, K, seed=5)
    fc1 = R.make_linear(K, N1, 32, fp4=False, x_absmax=x.float().abs().amax(0), seed=6, mode="svd")
    q1 = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=False)
    h = R.ref_gemm(q1, fc1, M=M, act="gelu")
    fc2 = R.make_linear(N1, K, 32, fp4=False, x_absmax=h.abs().amax(0).clamp(min=1e-3), seed=7, mode="svd")
    q2 = R.ref_requantize(h, fc2, M_pad=q1.codes.shape[0], unsigned=True)
    y = R.ref_gemm(q2, fc2, M=M)
    m1, m2 = H.to_module(fc1), H.to_module(fc2)
    m2.act_unsigned = True
    got = fused_gelu_mlp(x.cuda().view(1, M, K), m1, m2).float().cpu().view(M, K)
    assert R.rel_l2(got, y) <= 2e-2


@pytest.mark.parametrize("precision", ["nvfp4", "int4"])
def test_mlp_chain_config2_full_size_properties(precision):
    """The FLUX MLP chain at full size (M=4608, 3072 -> 12288 -> 3072, rank 32, random packed weights), through
    properties that need no oracle run: the chain is repeatable bit for bit, and rows are independent - the first 512
    rows computed alone agree with the same rows of the full call within the path's tolerance (relative L2 <= 1e-2; the
    fused LoRA-down sums its partials in a tile order that depends on M, so 4-bit codes of fc2's input may differ by one
    step here and there)."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.models.random_init import random_w4a4_linear

    def random_linear(i, o, r, prec, seed):
        return random_w4a4_linear(i, o, r, prec, True, torch.Generator(device="cuda").manual_seed(seed), bias_std=0.02, int4_scale=2.0 ** -7)
    from nunchaku_b200.ops import fused_gelu_mlp

    M, Hd = 4608, 3072
    fc1, fc2 = random_linear(Hd, 4 * Hd, 32, precision, 1), random_linear(4 * Hd, Hd, 32, precision, 2)
    if precision == "int4":
        fc2.act_unsigned = True      # fc1's requantising epilogue emits shifted unsigned codes
    x = torch.randn(1, M, Hd, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(3))
    y1 = fused_gelu_mlp(x, fc1, fc2)
    y2 = fused_gelu_mlp(x, fc1, fc2)
    ys = fused_gelu_mlp(x[:, :512].contiguous(), fc1, fc2)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.isfinite(y1).all() and torch.equal(y1, y2)
    assert R.rel_l2(ys.float().cpu().view(512, Hd), y1[:, :512].float().cpu().view(512, Hd)) <= 1e-2
