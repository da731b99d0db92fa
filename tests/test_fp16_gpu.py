"""The fp16 configuration of the path (the reference's GEMMConfig_W4A4_FP16, src/kernels/zgemm/gemm_w4a4.cu:17-31): the same
kernels compiled for fp16 activations, smoothing factors, LoRA weights, biases, INT4 scales and outputs, against the CPU
oracle run with the same type.

Tolerances: the quantiser's codes and scale bytes are bit-exact away from rounding ties; fp16 outputs carry three more
mantissa bits than bf16 ones, so the GEMM is held to 1e-3 where the bf16 tests use 4e-3."""
import pytest
import torch

import helpers as H
from oracle import layouts as L
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu

F16 = torch.float16
LORA_RTOL = 2e-5
REL_L2_F16 = 1e-3


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("layout", ["native", "reference"])
@pytest.mark.parametrize("M,K,Rk", [(256, 128, 32), (300, 512, 32), (1, 384, 48), (520, 1024, 64), (256, 256, 160)])
def test_fp16_quantize_matches_oracle(M, K, Rk, fp4, layout):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    x = R.make_activations(M, K, seed=M + K, dtype=F16)
    lin = R.make_linear(K, 128, Rk, fp4=fp4, x_absmax=x.float().abs().amax(0).clamp(min=1e-3), seed=3, dtype=F16)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    codes, scales, lora = svdq_quantize_w4a4_act_fuse_lora_cuda(
        x.cuda(), lora_down=L.ref_pack_lora_down(lin.lora_down).cuda(), smooth=L.ref_pack_vector(lin.smooth).cuda(),
        fp4=fp4, layout=_lib.LAYOUT_NATIVE if layout == "native" else _lib.LAYOUT_REFERENCE,
    )
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert scales.dtype == (torch.float8_e4m3fn if fp4 else F16)
    ec, es, el = H.pack_quant_out(q, layout)
    got = H.unpack_quant_out(codes, scales, lora, K, fp4, layout)
    H.assert_codes_match(got.codes, q)
    view = torch.uint8 if fp4 else torch.int16
    assert torch.equal(scales.cpu().view(view), es.view(view)), "scale bytes differ from the oracle"
    err = (lora.cpu() - el).abs().max().item()
    assert err <= LORA_RTOL * max(el.abs().max().item(), 1.0) + 1e-6


@pytest.mark.parametrize("fp4", [True, False])
def test_fp16_quantize_fuse_glu(fp4):
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    M, K = 300, 256
    x = (torch.randn(M, 2 * K, generator=torch.Generator().manual_seed(1)) * 1.5).to(F16)
    lin = R.make_linear(K, 128, 32, fp4=fp4, seed=5, dtype=F16)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4, fuse_glu=True)
    codes, scales, lora = svdq_quantize_w4a4_act_fuse_lora_cuda(
        x.cuda(), lora_down=L.ref_pack_lora_down(lin.lora_down).cuda(), smooth=L.ref_pack_vector(lin.smooth).cuda(),
        fp4=fp4, fuse_glu=True)
    got = H.unpack_quant_out(codes, scales, lora, K, fp4, "native")
    # the gate goes through ex2.approx / rcp.approx on the GPU and an exact sigmoid in the oracle: nearly all codes equal
    assert (got.codes == q.codes).float().mean().item() >= 0.99
    assert R.rel_l2(R.dequant_act(got), R.dequant_act(q)) <= 6e-3
    assert R.rel_l2(got.lora_act, q.lora_act) <= 2e-3


def _gemm(q, lin, M, act_unsigned=False, fuse_silu=False):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    sd = {k: v.cuda() for k, v in H.packed_params(lin).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.full((M, lin.N), float("nan"), dtype=F16, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd["qweight"], out=out, ascales=scales, wscales=sd["wscales"], lora_act_in=lora,
                        lora_up=sd["proj_up"], bias=sd.get("bias"), fp4=lin.fp4, alpha=lin.wtscale if lin.fp4 else 1.0,
                        wcscales=sd.get("wcscales"), fuse_silu=fuse_silu, act_unsigned=act_unsigned, act_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    return out.float().cpu()


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("M,K,N,Rk", [(256, 256, 384, 32), (300, 512, 640, 16), (1024, 1024, 3072, 32)])
def test_fp16_gemm_matches_oracle(M, K, N, Rk, fp4):
    x = R.make_activations(M, K, seed=M + N, dtype=F16)
    lin = R.make_linear(K, N, Rk, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=M + N + 1, mode="svd", wcscales=fp4, dtype=F16)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    exp = R.ref_gemm(q, lin, M=M)
    got = _gemm(q, lin, M)
    assert not torch.isnan(got).any()
    # INT4: fp16(code * fp16 scale) rounds (14 significant bits into 11), once per operand
    assert R.rel_l2(got, exp) <= (REL_L2_F16 if fp4 else 2e-3)
    got_silu = _gemm(q, lin, M, fuse_silu=True)
    assert R.rel_l2(got_silu, R.ref_gemm(q, lin, M=M, act="silu")) <= 2e-3


def test_fp16_output_saturates_instead_of_overflowing():
    """Values beyond the fp16 range come out as +-65504 (the reference clamps its fp16 output, gemm_base.cuh:686-693)."""
    M, K, N = 256, 128, 128
    x = R.make_activations(M, K, seed=2, dtype=F16)
    lin = R.make_linear(K, N, 16, fp4=True, x_absmax=x.float().abs().amax(0), seed=4, dtype=F16)
    lin.bias = torch.full((N,), 65000.0, dtype=F16)
    lin.wcscales = torch.full((N,), 1.0, dtype=F16)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=True)
    lin.bias[::2] = -65000.0
    lin.wtscale = lin.wtscale * 3000.0     # pushes many sums beyond 65504
    got = _gemm(q, lin, M)
    assert torch.isfinite(got).all() and got.abs().max().item() == 65504.0
    exp = R.ref_gemm(q, lin, M=M).clamp(-65504.0, 65504.0)
    assert R.rel_l2(got, exp) <= 2e-3


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("M,K,N,R1,R2", [(300, 256, 384, 32, 32), (256, 512, 1024, 32, 16), (256, 128, 256, 16, 96)])
def test_fp16_gemm_gelu_requant(M, K, N, R1, R2, fp4):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    torch.manual_seed(0)
    x = R.make_activations(M, K, seed=M + N, dtype=F16)
    fc1 = R.make_linear(K, N, R1, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=M + 1, mode="svd", wcscales=fp4, dtype=F16)
    fc2 = R.make_linear(N, 256, R2, fp4=fp4, x_absmax=torch.rand(N) + 0.5, seed=M + 2, dtype=F16)
    q = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=fp4)
    M_pad = q.codes.shape[0]
    sd1 = {k: v.cuda() for k, v in H.packed_params(fc1).items()}
    sd2 = {k: v.cuda() for k, v in H.packed_params(fc2).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]
    out = torch.full((M, N), float("nan"), dtype=F16, device="cuda")
    qout = torch.zeros(M_pad, N // 2, dtype=torch.uint8, device="cuda")
    osc = (torch.zeros(N // 16, M_pad, dtype=torch.float8_e4m3fn, device="cuda") if fp4
           else torch.zeros(N // 64, M_pad, dtype=F16, device="cuda"))
    la2 = torch.full((M_pad, R2), float("nan"), dtype=torch.float32, device="cuda")
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd1["qweight"], out=out, qout=qout, ascales=scales, wscales=sd1["wscales"], oscales=osc,
                        lora_act_in=lora, lora_up=sd1["proj_up"], lora_down=sd2["proj_down"], lora_act_out=la2,
                        bias=sd1["bias"], smooth_factor=sd2["smooth_factor"], fp4=fp4, alpha=fc1.wtscale if fp4 else 1.0,
                        wcscales=sd1.get("wcscales"), act_layout=_lib.LAYOUT_NATIVE, out_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    got = H.unpack_quant_out(qout, osc, la2, N, fp4, "native")
    got.unsigned = not fp4
    y = R.ref_gemm(q, fc1, M=M, act="gelu")
    assert R.rel_l2(out.float().cpu(), y) <= 2e-3
    # given the kernel's own fp16 tile: codes and scales bit-exact, LoRA-down tight
    exp = R.ref_requantize(out.float().cpu(), fc2, M_pad=M_pad, unsigned=not fp4)
    H.assert_codes_match(got.codes, exp, rows=slice(0, M), what="requantised codes (given the kernel's own output)")
    view = torch.uint8 if fp4 else torch.int16
    assert torch.equal(got.scales[:, :M].contiguous().view(view), exp.scales[:, :M].contiguous().view(view))
    err = (got.lora_act[:M] - exp.lora_act[:M]).abs().max().item()
    assert err <= 2e-5 * max(exp.lora_act.abs().max().item(), 1.0) + 1e-6


@pytest.mark.parametrize("precision", ["nvfp4", "int4"])
def test_fp16_module_and_fused_mlp(precision):
    """SVDQW4A4Linear(torch_dtype=float16) end to end and through fused_gelu_mlp, against the oracle chain."""
    from nunchaku_b200.ops import fused_gelu_mlp

    fp4 = precision == "nvfp4"
    M, K, N1 = 300, 256, 1024
    x = R.make_activations(M, K, seed=5, dtype=F16)
    fc1 = R.make_linear(K, N1, 32, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=6, mode="svd", dtype=F16)
    q1 = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=fp4)
    h = R.ref_gemm(q1, fc1, M=M, act="gelu")
    fc2 = R.make_linear(N1, K, 32, fp4=fp4, x_absmax=(h.abs().amax(0) + (0.0 if fp4 else 0.171875)).clamp(min=1e-3), seed=7,
                        mode="svd", dtype=F16)
    q2 = R.ref_requantize(h, fc2, M_pad=q1.codes.shape[0], unsigned=not fp4)
    y = R.ref_gemm(q2, fc2, M=M)
    m1, m2 = H.to_module(fc1), H.to_module(fc2, act_unsigned=not fp4)
    assert m1.proj_down.dtype == F16
    got1 = m1(x.cuda().view(1, M, K)).float().cpu().view(M, N1)
    assert R.rel_l2(got1, R.ref_gemm(q1, fc1, M=M)) <= 3e-3
    got = fused_gelu_mlp(x.cuda().view(1, M, K), m1, m2)
    assert got.dtype == F16
    assert R.rel_l2(got.float().cpu().view(M, K), y) <= 2e-2
