"""Measure the tensor-pipe rate of tcgen05.mma on this GPU with operands resident in shared memory /
TMEM (no loads): the measured dense peak that a GEMM's tensor-pipe fraction is judged against.

    python -m nunchaku_b200.peak_probe
"""
from __future__ import annotations

import ctypes
import json

import torch

from . import _lib

KINDS = {"mxf4nvf4": (0, 64), "tf32": (1, 8), "i8": (2, 32), "f16": (3, 16)}   # f16: pair probe only


def mma_rate(kind: str, n: int, iters: int = 2000, cps_per_group: int = 0, sf_buffers: int = 1, grid: int | None = None,
             sfb_step: int = 8, commit_every: bool = False, poll_warps: int = 0):
    lib = _lib.load()
    lib.svdq_probe_mma_rate.restype = ctypes.c_int32
    lib.svdq_probe_mma_rate.argtypes = [ctypes.c_int32] * 6 + [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int32] * 3
    dev = torch.device("cuda", torch.cuda.current_device())
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    grid = grid or sms
    cyc = torch.zeros(grid * 2, dtype=torch.int64, device=dev)
    code, k = KINDS[kind]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    def launch():
        _lib.check(lib.svdq_probe_mma_rate(code, n, iters, cps_per_group, sf_buffers, grid, cyc.data_ptr(),
                                           torch.cuda.current_stream(dev).cuda_stream, sfb_step, int(commit_every), poll_warps))

    for rep in range(2):
        e0.record()
        launch()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    c = cyc.view(grid, 2).double().mean(0)
    flops = 2.0 * 128 * n * k * 4 * iters * grid
    return {
        "kind": kind, "n": n, "cps_per_group": cps_per_group, "sf_buffers": sf_buffers, "sfb_step": sfb_step,
        "commit_every": commit_every, "poll_warps": poll_warps,
        "cycles_per_mma_issue": c[0].item() / (4 * iters), "cycles_per_mma": c[1].item() / (4 * iters),
        "tflops": flops / (ms * 1e-3) / 1e12, "ms": ms,
        "sm_mhz": c[1].item() / (ms * 1e3),   # SM clock during the loop: its cycles over its duration
    }


def mma_rate_pair(kind: str, n: int, iters: int = 2000, grid: int | None = None, cps_per_group: int = 0):
    """MMA rate of a CTA pair (cta_group::2, M = 256): cycles per MMA and the whole-GPU TFLOP/s."""
    lib = _lib.load()
    lib.svdq_probe_mma_rate_pair.restype = ctypes.c_int32
    lib.svdq_probe_mma_rate_pair.argtypes = [ctypes.c_int32] * 4 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32]
    dev = torch.device("cuda", torch.cuda.current_device())
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    grid = grid or (sms // 2) * 2
    cyc = torch.zeros(grid * 2, dtype=torch.int64, device=dev)
    code, k = KINDS[kind]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(2):
        e0.record()
        _lib.check(lib.svdq_probe_mma_rate_pair(code, n, iters, grid, cyc.data_ptr(), torch.cuda.current_stream(dev).cuda_stream,
                                                cps_per_group))
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    c = cyc.view(grid, 2)[0::2].double().mean(0)     # the issuing CTAs
    flops = 2.0 * 256 * n * k * 4 * iters * (grid // 2)
    return {"kind": kind, "n": n, "pair": True, "cps_per_group": cps_per_group, "cycles_per_mma_issue": c[0].item() / (4 * iters),
            "cycles_per_mma": c[1].item() / (4 * iters), "tflops": flops / (ms * 1e-3) / 1e12, "ms": ms}


def main():
    out = []
    for kind, n in [("mxf4nvf4", 256), ("mxf4nvf4", 192), ("mxf4nvf4", 128), ("i8", 256), ("i8", 128), ("tf32", 192)]:
        out.append(mma_rate(kind, n))
    for cps, bufs in [(4, 1), (12, 1), (12, 2)]:
        out.append(mma_rate("mxf4nvf4", 192, cps_per_group=cps, sf_buffers=bufs))
    for r in out:
        print(json.dumps(r))
    assert _lib.device_status() == (0, 0)


if __name__ == "__main__":
    main()
