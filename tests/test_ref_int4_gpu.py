"""Parity against the reference ITSELF: its INT4 (bf16) W4A4 kernels, compiled from the reference tree into
``oracle/_ref/libnunchaku_ref_int4.so`` (``python -m oracle.build_ref``), run on this GPU next to this library's kernels
and to the CPU oracle, on the same seeded inputs.

What is pinned here:
* the oracle's quantiser arithmetic (smoothing division, bf16 roundings, absmax, scale, round-to-nearest-even codes,
  packed layouts of codes / scales / low-rank activations) against the reference kernel's bytes;
* this library's INT4 quantiser bytes against the reference kernel's bytes (reference layout);
* GEMM epilogues (bias, LoRA-up, SiLU, GELU + u4 requantisation + LoRA-down, RMSNorm + RoPE, ReLU linear attention)
  against the reference's outputs, within the tolerance its own bf16 accumulation allows.
The reference's NVFP4 kernels cannot run on sm_100 (they trap outside sm_120a), so NVFP4 shares this pin only through
the code paths common to both precisions (smoothing, bf16 rounding, absmax, layouts of the low-rank tensors).
Tolerances: the reference rounds its accumulator to bf16 after every 64-k group (gemm_base.cuh:367-409) and evaluates
rcp / division with approximate instructions, so bytes can differ on ties and GEMM outputs agree to about 1e-2.
"""
import pytest
import torch

import helpers as H
import ref_int4 as REF
from oracle import layouts as L
from oracle import svdq_ref as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not REF.available(), reason="oracle/_ref has not been built")]

DEV = "cuda:0"


def _quant_inputs(M, K, Rk, seed, glu=False):
    x = R.make_activations(M, 2 * K if glu else K, seed=seed)
    if glu:
        v = (x[:, 0::2].float() * (x[:, 1::2].float() * torch.sigmoid(x[:, 1::2].float())).to(torch.bfloat16).float()).to(torch.bfloat16)
    else:
        v = x
    lin = R.make_linear(K, 128, Rk, fp4=False, x_absmax=v.float().abs().amax(0).clamp(min=1e-3), seed=seed + 1)
    return x, lin


@pytest.mark.parametrize("M,K,Rk", [(256, 128, 16), (300, 512, 32), (1000, 1024, 64), (4096, 3072, 32)])
def test_quantiser_bytes_match_the_reference_kernel(M, K, Rk):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    x, lin = _quant_inputs(M, K, Rk, seed=M + K)
    sm, ld = L.ref_pack_vector(lin.smooth).to(DEV), L.ref_pack_lora_down(lin.lora_down).to(DEV)
    rc, rs, rl = REF.quantize(x.to(DEV), sm, ld)
    oc, os_, ol = svdq_quantize_w4a4_act_fuse_lora_cuda(x.to(DEV), lora_down=ld, smooth=sm, fp4=False, layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    # this library vs the reference kernel, raw bytes in the reference's own layout
    assert torch.equal(rs.view(torch.int16), os_.view(torch.int16)), "scale bytes differ from the reference kernel"
    ref_q = H.unpack_quant_out(rc.view(torch.uint8), rs, rl, K, False, "reference")
    our_q = H.unpack_quant_out(oc, os_, ol, K, False, "reference")
    diff = (ref_q.codes[:M] != our_q.codes[:M])
    # same instruction sequence for the scale's reciprocal and the rounding: the codes are the reference kernel's, bit for bit
    assert not diff.any(), f"{int(diff.sum())} of {diff.numel()} codes differ from the reference kernel"
    assert torch.equal(rc.view(torch.uint8), oc), "packed code bytes differ from the reference kernel"
    assert not ref_q.codes[M:].any() and not our_q.codes[M:].any()
    tol = 1e-4 * max(ref_q.lora_act.abs().max().item(), 1.0)
    assert (ref_q.lora_act - our_q.lora_act).abs().max().item() <= tol
    # the CPU oracle vs the reference kernel: this is what pins the oracle's arithmetic
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    assert torch.equal(q.scales.view(torch.int16), ref_q.scales.view(torch.int16)), "oracle scales differ from the reference kernel"
    H.assert_codes_match(ref_q.codes, q, rows=slice(0, M), what="codes of the reference kernel")
    assert (q.lora_act - ref_q.lora_act).abs().max().item() <= tol


@pytest.mark.parametrize("M,K,Rk", [(300, 512, 32), (1000, 1024, 64), (2048, 3072, 32)])
def test_fp16_quantiser_bytes_match_the_reference_kernel(M, K, Rk):
    """The fp16 configuration (GEMMConfig_W4A4_FP16): this library's quantiser and the oracle against the reference's fp16
    INT4 kernel.  The reference divides by the smoothing factor with rcp.approx + one rounding (cuda_fp16.hpp, __hdiv); so
    does the fp16 build of this library, while the oracle divides exactly: a handful of values within 2^-23 of an fp16
    rounding boundary may differ there."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    x = R.make_activations(M, K, seed=M + K, dtype=torch.float16)
    lin = R.make_linear(K, 128, Rk, fp4=False, x_absmax=x.float().abs().amax(0).clamp(min=1e-3), seed=M + 1, dtype=torch.float16)
    sm, ld = L.ref_pack_vector(lin.smooth).to(DEV), L.ref_pack_lora_down(lin.lora_down).to(DEV)
    rc, rs, rl = REF.quantize(x.to(DEV), sm, ld)
    oc, os_, ol = svdq_quantize_w4a4_act_fuse_lora_cuda(x.to(DEV), lora_down=ld, smooth=sm, fp4=False, layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.equal(rs.view(torch.int16), os_.view(torch.int16)), "scale bytes differ from the reference kernel"
    assert torch.equal(rc.view(torch.uint8), oc), "packed code bytes differ from the reference kernel"
    ref_q = H.unpack_quant_out(rc.view(torch.uint8), rs, rl, K, False, "reference")
    our_q = H.unpack_quant_out(oc, os_, ol, K, False, "reference")
    tol = 1e-4 * max(ref_q.lora_act.abs().max().item(), 1.0)
    assert (ref_q.lora_act - our_q.lora_act).abs().max().item() <= tol
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    same_scales = (q.scales.view(torch.int16) == ref_q.scales.view(torch.int16)).float().mean().item()
    assert same_scales >= 0.9999, f"oracle scales vs the reference kernel: {same_scales}"
    bad = (ref_q.codes[:M] != q.codes[:M]) & ~q.tie[:M]
    assert bad.float().mean().item() <= 1e-5, f"{int(bad.sum())} oracle codes differ from the reference kernel away from ties"


def test_fp16_gemm_against_the_reference_kernel():
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    M, K, N = 300, 512, 384
    x = R.make_activations(M, K, seed=7, dtype=torch.float16)
    lin = R.make_linear(K, N, 32, fp4=False, x_absmax=x.float().abs().amax(0), seed=8, mode="svd", dtype=torch.float16)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    codes, scales, lora, p = _packed(lin, q)
    out_ref = torch.empty(M, N, dtype=torch.float16, device=DEV)
    REF.gemm(codes.view(torch.int8), p["qweight"], scales, p["wscales"], out=out_ref, lora_act_in=lora, lora_up=p["proj_up"],
             bias=p["bias"])
    out = torch.empty(M, N, dtype=torch.float16, device=DEV)
    svdq_gemm_w4a4_cuda(act=codes, wgt=p["qweight"], out=out, ascales=scales, wscales=p["wscales"], lora_act_in=lora,
                        lora_up=p["proj_up"], bias=p["bias"], fp4=False, act_layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    y = R.ref_gemm(q, lin, M=M)
    e_ref, e_our = R.rel_l2(out_ref.float().cpu(), y), R.rel_l2(out.float().cpu(), y)
    assert e_ref <= 5e-3, f"reference kernel vs fp32 oracle: {e_ref}"      # fp16 accumulation over K/64 groups
    assert e_our <= 2e-3, f"this library vs fp32 oracle: {e_our}"
    assert R.rel_l2(out.float().cpu(), out_ref.float().cpu()) <= 5e-3


def test_quantiser_edge_values_match_the_reference_kernel():
    """Zero rows and groups, negative zero, huge and tiny magnitudes, rounding ties."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    M, K = 256, 256
    g = torch.Generator().manual_seed(9)
    x = torch.randn(M, K, generator=g)
    x[3] = 0.0
    x[5, :64] = 0.0
    x[7, 64:128] = -0.0
    x[9, 40] = 3.0e4
    x[10] *= 1e-5
    x[11, :64] = torch.arange(64).float() * 0.5 - 16.0
    x[13, :64] = torch.tensor([0.5, 1.5, 2.5, 3.5, 4.5, 5.5, 6.5, 7.0] * 8)   # exact .5 ties when the scale is 1
    x = x.to(torch.bfloat16)
    lin = R.make_linear(K, 128, 32, fp4=False, x_absmax=None, seed=3)
    sm, ld = L.ref_pack_vector(lin.smooth).to(DEV), L.ref_pack_lora_down(lin.lora_down).to(DEV)
    rc, rs, rl = REF.quantize(x.to(DEV), sm, ld)
    oc, os_, ol = svdq_quantize_w4a4_act_fuse_lora_cuda(x.to(DEV), lora_down=ld, smooth=sm, fp4=False, layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert torch.equal(rs.view(torch.int16), os_.view(torch.int16))
    assert torch.equal(rc.view(torch.uint8), oc), "packed code bytes differ from the reference kernel"
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    ref_q = H.unpack_quant_out(rc.view(torch.uint8), rs, rl, K, False, "reference")
    assert torch.equal(q.scales.view(torch.int16), ref_q.scales.view(torch.int16))
    H.assert_codes_match(ref_q.codes, q, what="codes of the reference kernel")


def test_glu_quantiser_matches_the_reference_kernel():
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    M, K = 520, 512
    x, lin = _quant_inputs(M, K, 32, seed=5, glu=True)
    sm, ld = L.ref_pack_vector(lin.smooth).to(DEV), L.ref_pack_lora_down(lin.lora_down).to(DEV)
    rc, rs, rl = REF.quantize(x.to(DEV), sm, ld, fuse_glu=True)
    oc, os_, ol = svdq_quantize_w4a4_act_fuse_lora_cuda(x.to(DEV), lora_down=ld, smooth=sm, fp4=False, fuse_glu=True,
                                                        layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    # both evaluate the sigmoid with ex2.approx / rcp.approx: the bytes should agree almost everywhere
    assert (rs.view(torch.int16) == os_.view(torch.int16)).float().mean().item() >= 0.999
    assert (rc.view(torch.uint8) == oc).float().mean().item() >= 0.999
    assert R.rel_l2(ol.cpu(), rl.cpu()) <= 1e-3


def _gemm_problem(M, K, N, Rk, seed):
    x = R.make_activations(M, K, seed=seed)
    lin = R.make_linear(K, N, Rk, fp4=False, x_absmax=x.float().abs().amax(0), seed=seed + 1, mode="svd")
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=False)
    return x, lin, q


def _packed(lin, q):
    codes, scales, lora = [t.to(DEV) for t in H.pack_quant_out(q, "reference")]
    p = {k: v.to(DEV) for k, v in H.packed_params(lin).items()}
    return codes, scales, lora, p


@pytest.mark.parametrize("M,K,N,silu", [(300, 512, 384, False), (1024, 3072, 3072, False), (512, 256, 256, True)])
def test_gemm_against_the_reference_kernel(M, K, N, silu):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    x, lin, q = _gemm_problem(M, K, N, 32, seed=M + N)
    codes, scales, lora, p = _packed(lin, q)
    out_ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    REF.gemm(codes.view(torch.int8), p["qweight"], scales, p["wscales"], out=out_ref, lora_act_in=lora, lora_up=p["proj_up"],
             bias=p["bias"], fuse_silu=silu)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    svdq_gemm_w4a4_cuda(act=codes, wgt=p["qweight"], out=out, ascales=scales, wscales=p["wscales"], lora_act_in=lora,
                        lora_up=p["proj_up"], bias=p["bias"], fuse_silu=silu, fp4=False, act_layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    y = R.ref_gemm(q, lin, M=M, act="silu" if silu else None)
    e_ref, e_our = R.rel_l2(out_ref.float().cpu(), y), R.rel_l2(out.float().cpu(), y)
    assert e_ref <= 1.5e-2, f"reference kernel vs fp32 oracle: {e_ref}"      # bf16 accumulation over K/64 groups
    assert e_our <= 4e-3, f"this library vs fp32 oracle: {e_our}"
    assert R.rel_l2(out.float().cpu(), out_ref.float().cpu()) <= 1.5e-2


def test_gelu_requant_against_the_reference_kernel():
    """fc1 -> GELU -> +0.171875 -> / smooth_next -> u4 codes, and the next layer's LoRA-down (launch_impl.cuh:282-309)."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    M, K, N = 512, 512, 1024
    x, lin, q = _gemm_problem(M, K, N, 32, seed=21)
    nxt = R.make_linear(N, 128, 32, fp4=False, x_absmax=None, seed=23)
    codes, scales, lora, p = _packed(lin, q)
    nsm, nld = L.ref_pack_vector(nxt.smooth).to(DEV), L.ref_pack_lora_down(nxt.lora_down).to(DEV)

    def run(fn, layout_kw):
        qout = torch.empty(M, N // 2, dtype=torch.uint8, device=DEV)
        osc = torch.empty(N // 64, M, dtype=torch.bfloat16, device=DEV)
        la = torch.empty(M, 32, dtype=torch.float32, device=DEV)
        fn(qout, osc, la)
        torch.cuda.synchronize()
        out = H.unpack_quant_out(qout, osc, la, N, False, "reference")
        out.unsigned = True
        return out

    r = run(lambda qo, os_, la: REF.gemm(codes.view(torch.int8), p["qweight"], scales, p["wscales"], qout=qo.view(torch.int8),
                                         oscales=os_, lora_act_in=lora, lora_up=p["proj_up"], lora_down=nld, lora_act_out=la,
                                         bias=p["bias"], smooth_factor=nsm), None)
    o = run(lambda qo, os_, la: svdq_gemm_w4a4_cuda(act=codes, wgt=p["qweight"], qout=qo, ascales=scales, wscales=p["wscales"],
                                                    oscales=os_, lora_act_in=lora, lora_up=p["proj_up"], lora_down=nld,
                                                    lora_act_out=la, bias=p["bias"], smooth_factor=nsm, fp4=False,
                                                    act_layout=_lib.LAYOUT_REFERENCE, out_layout=_lib.LAYOUT_REFERENCE), None)
    assert _lib.device_status() == (0, 0)
    want = R.ref_requantize(R.ref_gemm(q, lin, M=M, act="gelu"), nxt, M_pad=M, unsigned=True)
    dw, dr, do = R.dequant_act(want), R.dequant_act(r), R.dequant_act(o)
    assert R.rel_l2(dr, dw) <= 3e-2, f"reference kernel vs oracle {R.rel_l2(dr, dw)}"
    assert R.rel_l2(do, dw) <= 2e-2, f"this library vs oracle {R.rel_l2(do, dw)}"
    assert R.rel_l2(do, dr) <= 3e-2
    assert R.rel_l2(r.lora_act, want.lora_act) <= 2e-2 and R.rel_l2(o.lora_act, want.lora_act) <= 1e-2


def _rotary_packed(M, seed):
    """cos / sin [M, 64] and the reference's packed tensor [1, M, 128] (layout of pack_rotemb, embeddings.py:88-120)."""
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(M, 64, generator=g) * 6.28
    cos, sin = ang.cos(), ang.sin()
    t = torch.stack([sin, cos], dim=-1).reshape(1, M, 64, 1, 2)          # (sin, cos) per pair, embeddings.py:36-39
    t = t.reshape(1, M // 16, 16, 16, 8).permute(0, 1, 3, 2, 4)
    t = t.reshape(1, M // 16, 16, 2, 8, 4, 2).permute(0, 1, 2, 4, 5, 3, 6).contiguous().view(1, M, 128)
    return cos, sin, t


def test_rmsnorm_rope_against_the_reference_kernel():
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    M, K, heads = 512, 512, 2
    N = 3 * heads * 128
    x, lin, q = _gemm_problem(M, K, N, 32, seed=31)
    codes, scales, lora, p = _packed(lin, q)
    g = torch.Generator().manual_seed(5)
    wq = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    wk = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    cos, sin, packed = _rotary_packed(M, 7)
    out_ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    REF.gemm(codes.view(torch.int8), p["qweight"], scales, p["wscales"], out=out_ref, lora_act_in=lora, lora_up=p["proj_up"],
             bias=p["bias"], norm_q=wq.to(DEV), norm_k=wk.to(DEV), rotary_emb=packed.to(DEV))
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    svdq_gemm_w4a4_cuda(act=codes, wgt=p["qweight"], out=out, ascales=scales, wscales=p["wscales"], lora_act_in=lora,
                        lora_up=p["proj_up"], bias=p["bias"], norm_q=wq.to(DEV), norm_k=wk.to(DEV), rotary_emb=packed.to(DEV),
                        fp4=False, act_layout=_lib.LAYOUT_REFERENCE)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    y = R.ref_gemm(q, lin, M=M).to(torch.bfloat16)
    want = R.ref_qk_norm_rope(y, wq, wk, cos, sin, heads).float()
    assert R.rel_l2(out_ref.float().cpu(), want) <= 2e-2, R.rel_l2(out_ref.float().cpu(), want)
    assert R.rel_l2(out.float().cpu(), want) <= 6e-3, R.rel_l2(out.float().cpu(), want)
    assert R.rel_l2(out.float().cpu(), out_ref.float().cpu()) <= 2e-2


def test_linear_attention_against_the_reference_kernel():
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops import linearattn_vk_mul_q
    from nunchaku_b200.ops.gemm import svdq_gemm_w4a4_cuda

    B, tokens, heads, K = 2, 256, 8, 256
    M, N = B * tokens, 3 * heads * 32
    x, lin, q = _gemm_problem(M, K, N, 32, seed=41)
    codes, scales, lora, p = _packed(lin, q)

    def run(gemm_fn, mul_fn):
        vk = torch.empty(B, heads, 33, 32, dtype=torch.float32, device=DEV)
        o = torch.empty(B, tokens, N // 3, dtype=torch.bfloat16, device=DEV)
        gemm_fn(vk, o)
        relu_q = o.clone()
        mul_fn(o, vk)
        torch.cuda.synchronize()
        return vk.cpu(), relu_q.float().cpu(), o.float().cpu()

    r = run(lambda vk, o: REF.gemm(codes.view(torch.int8), p["qweight"], scales, p["wscales"], lora_act_in=lora, lora_up=p["proj_up"],
                                   bias=p["bias"], out_vk=vk, out_linearattn=o), REF.vk_mul_q)
    u = run(lambda vk, o: svdq_gemm_w4a4_cuda(act=codes, wgt=p["qweight"], ascales=scales, wscales=p["wscales"], lora_act_in=lora,
                                              lora_up=p["proj_up"], bias=p["bias"], out_vk=vk, out_linearattn=o, fp4=False,
                                              act_layout=_lib.LAYOUT_REFERENCE), linearattn_vk_mul_q)
    assert _lib.device_status() == (0, 0)
    y = R.ref_gemm(q, lin, M=M).to(torch.bfloat16)
    want, want_vk = R.ref_litela(y.view(B, tokens, N), heads)
    assert R.rel_l2(r[0], want_vk) <= 2e-2 and R.rel_l2(u[0], want_vk) <= 6e-3
    assert R.rel_l2(u[1], torch.relu(y.view(B, tokens, N)[..., : N // 3].float())) <= 4e-3
    assert R.rel_l2(r[2], want.float()) <= 3e-2 and R.rel_l2(u[2], want.float()) <= 1e-2
    assert R.rel_l2(u[2], r[2]) <= 3e-2
