"""Time of the FLUX MLP chain on the W4A4 path: fc1 (hidden -> 4 x hidden) with GELU, the next layer's LoRA-down and
its 4-bit quantisation fused into the GEMM epilogue, then fc2 (4 x hidden -> hidden).

    python -m nunchaku_b200.models.mlp_bench [--tokens 4608] [--hidden 3072] [--rank 32] [--precision nvfp4] [--steps 20]

Weights are random packed W4A4 parameters (``SVDQW4A4Linear.randomize_``-style: random codes, constant group scales,
N(0, 0.02) low-rank factors); activations N(0, 1) bf16.  Prints one JSON line: the chain's time (CUDA events over
``--steps`` back-to-back calls) and each kernel's own time, all in microseconds.  ``--only requant`` / ``--only plain``
launch just the requantising / the plain fc1 GEMM (for a profiler capture of that kernel alone).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _lib
from ..ops import fused_gelu_mlp
from ..ops.gemm import svdq_gemm_w4a4_cuda
from .linear import SVDQW4A4Linear


def random_linear(i: int, o: int, rank: int, precision: str, seed: int) -> SVDQW4A4Linear:
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = SVDQW4A4Linear(i, o, rank=rank, bias=True, precision=precision, device="cuda")
    with torch.no_grad():
        q.qweight.copy_(torch.randint(-128, 128, q.qweight.shape, device="cuda", dtype=torch.int16, generator=g).to(torch.int8))
        if precision == "nvfp4":
            q.wscales.copy_(torch.full(q.wscales.shape, 2.0 ** -7, device="cuda").to(torch.float8_e4m3fn))
        else:
            q.wscales.fill_(2.0 ** -7)
        q.smooth_factor.fill_(1.0)
        q.smooth_factor_orig.fill_(1.0)
        q.proj_down.copy_(torch.randn(q.proj_down.shape, device="cuda", generator=g) * 0.02)
        q.proj_up.copy_(torch.randn(q.proj_up.shape, device="cuda", generator=g) * 0.02)
        q.bias.copy_(torch.randn(q.bias.shape, device="cuda", generator=g) * 0.02)
    return q


def timed(fn, steps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4608)
    ap.add_argument("--hidden", type=int, default=3072)
    ap.add_argument("--rank", type=int, default=32)
    ap.add_argument("--precision", default="nvfp4", choices=["nvfp4", "int4"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--only", default=None, choices=[None, "requant", "plain"])
    args = ap.parse_args()
    M, H, fp4 = args.tokens, args.hidden, args.precision == "nvfp4"
    fc1 = random_linear(H, 4 * H, args.rank, args.precision, 1)
    fc2 = random_linear(4 * H, H, args.rank, args.precision, 2)
    x = torch.randn(1, M, H, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(0))

    q, s, la = fc1.quantize(x.view(M, H))
    M_pad = q.shape[0]
    qout = torch.empty(M_pad, 4 * H // 2, dtype=torch.uint8, device="cuda")
    if fp4:
        osc = torch.empty(4 * H // 16, M_pad, dtype=torch.float8_e4m3fn, device="cuda")
    else:
        osc = torch.empty(4 * H // 64, M_pad, dtype=torch.bfloat16, device="cuda")
    la2 = torch.empty(M_pad, args.rank, dtype=torch.float32, device="cuda")

    def fc1_requant():
        svdq_gemm_w4a4_cuda(act=q, wgt=fc1.qweight, qout=qout, ascales=s, wscales=fc1.wscales, oscales=osc, lora_act_in=la,
                            lora_up=fc1.proj_up, lora_down=fc2.proj_down, lora_act_out=la2, bias=fc1.bias,
                            smooth_factor=fc2.smooth_factor, fp4=fp4, alpha=fc1.wtscale, wcscales=fc1.wcscales, next_fp4=fp4)

    if args.only == "requant":
        us = timed(fc1_requant, args.steps)
        torch.cuda.synchronize()
        assert _lib.device_status() == (0, 0)
        print(json.dumps({"fc1_requant_gemm_us": round(us, 1), "tokens": M, "hidden": H, "rank": args.rank, "precision": args.precision}))
        return

    out1 = torch.empty(M, 4 * H, dtype=torch.bfloat16, device="cuda")
    out2 = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    if args.only == "plain":
        us = timed(lambda: fc1.forward_quant(q, s, la, out1), args.steps)
        torch.cuda.synchronize()
        assert _lib.device_status() == (0, 0)
        fl = 2.0 * M * H * 4 * H + 2.0 * M * 4 * H * args.rank
        print(json.dumps({"fc1_plain_gemm_us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "tokens": M, "hidden": H,
                          "rank": args.rank, "precision": args.precision}))
        return
    res = {
        "mlp_chain_us": timed(lambda: fused_gelu_mlp(x, fc1, fc2), args.steps),
        "fc1_quantize_us": timed(lambda: fc1.quantize(x.view(M, H)), args.steps),
        "fc1_requant_gemm_us": timed(fc1_requant, args.steps),
        "fc1_plain_gemm_us": timed(lambda: fc1.forward_quant(q, s, la, out1), args.steps),
        "fc2_gemm_us": timed(lambda: fc2.forward_quant(qout, osc, la2, out2), args.steps),
    }
    flop = 2.0 * M * H * 4 * H * 2 + 2.0 * M * args.rank * (H + 4 * H) * 2
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    print(json.dumps({**{k: round(v, 1) for k, v in res.items()}, "chain_tflops": round(flop / res["mlp_chain_us"] / 1e6, 1),
                      "tokens": M, "hidden": H, "rank": args.rank, "precision": args.precision,
                      "note": "each time includes the launch gap of a stand-alone launch (8-10 us)"}))


if __name__ == "__main__":
    main()
