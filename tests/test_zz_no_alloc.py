"""`svdq_gemm_w4a4_static_scratch`: the requantising NVFP4 GEMM for hosts that cannot pass a workspace
(a serving loop that split up its device memory at start-up and has no allocator to call per request, or one
that must not make allocation calls while serving).  The scratch then is an 8 MiB array inside the library.

Called through the C ABI with ctypes, twice in a row, and compared bit for bit with the regular entry point
(`svdq_gemm_w4a4` with a caller workspace): the kernel is deterministic, so the tolerance is zero.  This
file sorts last on purpose, so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

import helpers as H
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


def _problem(M, K, N, R1, R2, seed, fp4=True):
    x = R.make_activations(M, K, seed=seed)
    fc1 = R.make_linear(K, N, R1, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=seed + 1, mode="svd", wcscales=fp4)
    fc2 = R.make_linear(N, 256, R2, fp4=fp4, x_absmax=torch.rand(N) + 0.5, seed=seed + 2)
    q = R.ref_quantize(x, fc1.smooth, fc1.lora_down, fp4=fp4)
    return fc1, fc2, q


def _outputs(M, M_pad, N, R2, fp4=True):
    return dict(
        out=torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda"),
        qout=torch.full((M_pad, N // 2), 0xAA, dtype=torch.uint8, device="cuda"),
        osc=(torch.full((N // 16, M_pad), 0x55, dtype=torch.uint8, device="cuda") if fp4
             else torch.full((N // 64, M_pad), 7.0, dtype=torch.bfloat16, device="cuda")),
        la=torch.full((M_pad, R2), float("nan"), dtype=torch.float32, device="cuda"),
    )


def _args(lib, prepared, codes, scales, lora, o, sd2, M, M_pad, N, K, R1, R2, fp4=True):
    return lib.GemmArgs(
        act=codes.data_ptr(), ascales=scales.data_ptr(), lora_act_in=lora.data_ptr(), w=prepared.as_struct(),
        out=o["out"].data_ptr(), qout=o["qout"].data_ptr(), oscales=o["osc"].data_ptr(), lora_act_out=o["la"].data_ptr(),
        next_smooth=sd2["smooth_factor"].data_ptr(), next_lora_down=sd2["proj_down"].data_ptr(),
        workspace=None, workspace_bytes=0, M=M, M_pad=M_pad, N=N, K=K, R=R1, R_next=R2, fp4=int(fp4), act_unsigned=0,
        activation=lib.ACT_GELU, act_layout=lib.LAYOUT_NATIVE, out_layout=lib.LAYOUT_NATIVE, next_fp4=int(fp4),
    )


@pytest.mark.parametrize("fp4", [True, False])
def test_static_scratch_matches_workspace_entry_point(fp4):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops.gemm import cached_prepared_weights, svdq_gemm_w4a4_cuda

    M, K, N, R1, R2 = 700, 512, 1152, 32, 32
    fc1, fc2, q = _problem(M, K, N, R1, R2, seed=11, fp4=fp4)
    M_pad = q.codes.shape[0]
    sd1 = {k: v.cuda() for k, v in H.packed_params(fc1).items()}
    sd2 = {k: v.cuda() for k, v in H.packed_params(fc2).items()}
    codes, scales, lora = [t.cuda() for t in H.pack_quant_out(q, "native")]

    # regular entry point (the Python wrapper allocates the workspace through torch)
    ref = _outputs(M, M_pad, N, R2, fp4)
    svdq_gemm_w4a4_cuda(act=codes, wgt=sd1["qweight"], out=ref["out"], qout=ref["qout"], ascales=scales,
                        wscales=sd1["wscales"], oscales=ref["osc"].view(torch.float8_e4m3fn) if fp4 else ref["osc"], lora_act_in=lora,
                        lora_up=sd1["proj_up"], lora_down=sd2["proj_down"], lora_act_out=ref["la"], bias=sd1["bias"],
                        smooth_factor=sd2["smooth_factor"], fp4=fp4, alpha=fc1.wtscale, wcscales=sd1.get("wcscales"),
                        act_layout=_lib.LAYOUT_NATIVE, out_layout=_lib.LAYOUT_NATIVE)
    torch.cuda.synchronize()

    prepared = cached_prepared_weights(sd1["qweight"], sd1["wscales"], sd1["proj_up"], sd1["bias"], sd1.get("wcscales"),
                                       fc1.wtscale, [1.0, 1.0], fp4)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):   # the array keeps the previous call's partials: the second call must not care
        got = _outputs(M, M_pad, N, R2, fp4)
        a = _args(_lib, prepared, codes, scales, lora, got, sd2, M, M_pad, N, K, R1, R2, fp4)
        _lib.check(lib.svdq_gemm_w4a4_static_scratch(ctypes.byref(a), stream))
        torch.cuda.synchronize()
        assert _lib.device_status() == (0, 0)
        for k in ("out", "qout", "osc", "la"):
            assert torch.equal(got[k].view(torch.uint8), ref[k].view(torch.uint8)), f"{k} differs on call {call}"
    # and the result is right, not just equal: the low-rank output against the oracle on the kernel's own bf16 tile
    exp = R.ref_requantize(ref["out"].float().cpu(), fc2, M_pad=M_pad, unsigned=not fp4)
    assert (ref["la"].cpu()[:M] - exp.lora_act[:M]).abs().max().item() <= 2e-5 * max(exp.lora_act.abs().max().item(), 1.0) + 1e-6


def test_static_scratch_rejects_oversized_problems():
    from nunchaku_b200 import _lib

    lib = _lib.load()
    # 36 x 64 tiles on 148 CTAs with rank 64: 148 CTAs x 2 partials x 128 rows x 64 x 4 B = 9.7 MB > 8 MiB
    need = ctypes.c_size_t(0)
    a = _lib.GemmArgs(act=256, ascales=256, lora_act_in=256, w=_lib.PreparedWeights(wgt=256, wscales=256, lora_up=256, col_scale=256, col_bias=256),
                      out=None, qout=256, oscales=256, lora_act_out=256, next_smooth=256, next_lora_down=256,
                      workspace=None, workspace_bytes=0, M=4608, M_pad=4608, N=12288, K=3072, R=32, R_next=64, fp4=1,
                      act_unsigned=0, activation=_lib.ACT_GELU, act_layout=0, out_layout=0, next_fp4=1)
    _lib.check(lib.svdq_gemm_w4a4_workspace_bytes(ctypes.byref(a), ctypes.byref(need)))
    assert need.value > 8 << 20
    assert lib.svdq_gemm_w4a4_static_scratch(ctypes.byref(a), None) == _lib.SVDQ_ERR_INVALID_ARGUMENT
    assert b"scratch" in lib.svdq_last_error_string()
    a.fp4 = a.next_fp4 = 0      # the INT4 GEMM needs its partials plus the per-row normalisation scratch: larger still
    assert lib.svdq_gemm_w4a4_static_scratch(ctypes.byref(a), None) == _lib.SVDQ_ERR_INVALID_ARGUMENT
