#!/usr/bin/env python
"""Benchmark of the SVDQuant W4A4 linear hot path (quantise + 4-bit GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the NVFP4 FLUX single-block fused input projection, M=4608 tokens, K=3072, N=21504,
rank-32 low-rank branch, bf16 in / bf16 out, seeded synthetic data with the value distributions
of the benchmark description (N(0,1) activations with 1% outlier channels x20, N(0,0.02)
weights with the rank-32 SVD component removed, N(0,0.02) low-rank factors and bias).
One step = one pass of the path over one batch: activation quantiser + GEMM.  At N > 1 every rank
runs the same step on its own batch (the path shards along M without communication): weak scaling.
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, K, N, R = 4608, 3072, 21504, 32
METRIC = "W4A4 GEMM TFLOPS (NVFP4 W4A4+LoRA linear: activation quantiser + 4-bit GEMM)"
UNIT = "TFLOP/s"
FLOP_GEMM = 2.0 * M * N * K + 2.0 * M * N * R          # GEMM incl. LoRA-up
FLOP_STEP = FLOP_GEMM                                   # the metric counts GEMM FLOPs per pass of the path
QUANT_BYTES = 2 * M * K + M * K // 2 + M * K // 16 + 4 * M * R + 2 * K * R + 2 * K


# dram__bytes_read.sum + dram__bytes_write.sum of one full-size gemm_w4a4_kernel (NVFP4) launch (48.7 MB + 144.6 MB)
GEMM_DRAM_TRAFFIC = 48716544 + 144581632


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(M, K, generator=g, device=device)
    cols = torch.randperm(K, generator=g, device=device)[: max(1, (K + 99) // 100)]
    x[:, cols] *= 20.0
    return x.to(torch.bfloat16)


def build_layer(device, seed, x):
    from nunchaku_b200.models import SVDQW4A4Linear
    from nunchaku_b200.weights import svdquant_state_dict

    g = torch.Generator(device=device).manual_seed(seed + 1)
    W = torch.randn(N, K, generator=g, device=device) * 0.02
    b = torch.randn(N, generator=g, device=device) * 0.02
    torch.manual_seed(seed)
    sd = svdquant_state_dict(W, b, x.float().abs().amax(0), rank=R, precision="nvfp4", random_lowrank_std=0.02)
    m = SVDQW4A4Linear(K, N, rank=R, bias=True, precision="nvfp4", device=device)
    with torch.no_grad():
        for k, v in sd.items():
            getattr(m, k).copy_(v)
    return m


def cpu_oracle_setup(m):
    """Oracle (CPU restatement of the reference arithmetic) layer unpacked from the GPU layer's packed
    parameters.  Used only by the CPU-baseline leg and the reference arm."""
    from oracle import layouts as L
    from oracle import svdq_ref as Rf

    sd = {k: v.detach().cpu() for k, v in m.state_dict().items()}
    lin = Rf.Linear(
        K, N, R, True, L.ref_unpack_wgt_codes(sd["qweight"], K), L.ref_unpack_wmscales(sd["wscales"].view(torch.uint8)),
        L.ref_unpack_vector(sd["smooth_factor"]), L.ref_unpack_lora_down(sd["proj_down"]), L.ref_unpack_lora_up(sd["proj_up"]),
        L.ref_unpack_vector(sd["bias"]), float(sd["wtscale"].item()), L.ref_unpack_vector(sd["wcscales"]))
    wdeq = lin.dequant_weight()
    return lin, wdeq


def cpu_oracle_step(lin, wdeq, x_rows):
    """quantise + dequantise-matmul + epilogue on the CPU for `x_rows` (weights kept dequantised)."""
    from oracle import svdq_ref as Rf

    q = Rf.ref_quantize(x_rows, lin.smooth, lin.lora_down, fp4=True)
    a = Rf.dequant_act(q)[: x_rows.shape[0]]
    y = a @ wdeq.t()
    y = y * lin.wcscales.float() + lin.bias.float()
    y = y + q.lora_act[: x_rows.shape[0]] @ lin.lora_up.float().t()
    return y.to(torch.bfloat16)


def run_reference(args, rank):
    """Reference arm: the CPU restatement of the reference's arithmetic (the reference has no CPU
    implementation and its CUDA kernels have no sm_100 path), all host threads, bounded sample per step."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    from oracle import layouts as L  # noqa: F401  (fail early if the oracle is missing)
    x = make_inputs("cpu", 0)
    # build the same layer on the CPU (no GPU needed for this arm)
    m = build_layer("cpu", 0, x)
    lin, wdeq = cpu_oracle_setup(m)
    rows = 64
    t0 = time.perf_counter(); cpu_oracle_step(lin, wdeq, x[:rows]); probe = time.perf_counter() - t0
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = int(max(32, min(M, rows * budget / max(probe, 1e-3)))) // 32 * 32
    for _ in range(args.warmup):
        cpu_oracle_step(lin, wdeq, x[:rows])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_step(lin, wdeq, x[:rows])
    dt = (time.perf_counter() - t0) / args.steps
    val = FLOP_STEP * rows / M / dt / 1e12
    sample = f"{rows} of {M} rows per step (quantise + fp32 dequant-matmul + epilogue; weights kept dequantised)"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * M / rows, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4 (e2m1 x e2m1, ue4m3 group-16 scales), fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"NVFP4 W4A4+LoRA linear M={M} K={K} N={N} R={R} (FLUX single-block fused input projection)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shape", default=None, help="M,K,N override: a smaller case of the same path for profiler captures "
                    "(the default is the benchmark workload)")
    args = ap.parse_args()
    if args.shape:
        global M, K, N, FLOP_GEMM, FLOP_STEP, QUANT_BYTES
        M, K, N = (int(v) for v in args.shape.split(","))
        FLOP_GEMM = 2.0 * M * N * K + 2.0 * M * N * R
        FLOP_STEP = FLOP_GEMM
        QUANT_BYTES = 2 * M * K + M * K // 2 + M * K // 16 + 4 * M * R + 2 * K * R + 2 * K
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from nunchaku_b200 import distributed as D

    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return

    rank, world, local = D.init_from_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from nunchaku_b200 import _lib
    _lib.load()

    x = make_inputs(dev, rank)
    m = build_layer(dev, 0, x)
    xv = x.view(1, M, K)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

    def step():
        q, s, la = m.quantize(x)
        m.forward_quant(q, s, la, out)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    # ---- timed region: K steps, inputs resident in HBM; per-kernel events for the roofline figures
    # Per-kernel durations come from CUDA events inside the timed region, on a sample of its steps (every 4th, at
    # least 3): an event between two kernels costs a few microseconds of a 185 us step and keeps the second kernel's
    # launch from overlapping the first one's tail, so timing every launch would slow down what is being measured.
    stride = 4 if args.steps >= 12 else 1
    sampled = [i for i in range(args.steps) if i % stride == 0]
    ev = {i: [torch.cuda.Event(enable_timing=True) for _ in range(3)] for i in sampled}
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    D.barrier()
    torch.cuda.synchronize()
    e_start.record()
    for i in range(args.steps):
        if i in ev:
            ev[i][0].record()
            q, s, la = m.quantize(x)
            ev[i][1].record()
            m.forward_quant(q, s, la, out)
            ev[i][2].record()
        else:
            q, s, la = m.quantize(x)
            m.forward_quant(q, s, la, out)
    e_stop.record()
    torch.cuda.synchronize()
    D.barrier()
    ms_total = e_start.elapsed_time(e_stop)
    # keep the sampler alive for at least a few samples on very short regions
    if ms_total < 400:
        t_end = time.time() + 0.4
        while time.time() < t_end:
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_step = D.max_over_ranks(ms_total / args.steps, dev)
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in ev.values()) / len(ev)
    gemm_ms = sum(e[1].elapsed_time(e[2]) for e in ev.values()) / len(ev)
    status = _lib.device_status()
    if status != (0, 0):
        raise SystemExit(f"device status {status}: a bounded wait ran out")

    # ---- end to end through the public module API with host buffers
    # Every step copies its own input from pinned host memory and its own result back; HostPipeline puts the
    # two copies and the kernels on three streams with double-buffered device tensors, so consecutive steps
    # overlap (copy-in of i+1, compute of i, copy-out of i-1) as they would in a serving loop.
    from nunchaku_b200.host_pipeline import HostPipeline
    xh = [torch.empty(1, M, K, dtype=torch.bfloat16, pin_memory=True).copy_(x.cpu().view(1, M, K)) for _ in range(2)]
    oh = [torch.empty(M, N, dtype=torch.bfloat16, pin_memory=True) for _ in range(2)]
    pipe = HostPipeline(m, (1, M, K), (M, N), device=dev)

    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        pipe.submit(xh[i % 2], oh[i % 2])
    pipe.join()
    D.barrier()
    torch.cuda.synchronize()
    e_start.record()
    pipe.fork()
    for i in range(e2e_steps):
        pipe.submit(xh[i % 2], oh[i % 2])
    pipe.join()
    e_stop.record()
    torch.cuda.synchronize()
    if not torch.equal(oh[0], out.cpu()) or not torch.equal(oh[1], oh[0]):
        raise SystemExit("end-to-end result differs from the device-resident result")
    e2e_ms = D.max_over_ranks(e_start.elapsed_time(e_stop) / e2e_steps, dev)

    peaks, peak_kind = load_peaks()
    # FP4 has no entry in MEASURED_PEAKS.json: measure the tensor-pipe peak here, on this GPU, with the
    # library's operand-resident tcgen05.mma loop (kind::mxf4nvf4, M128 N256 K64 per instruction).
    from nunchaku_b200.peak_probe import mma_rate
    fp4_peak = mma_rate("mxf4nvf4", 256, iters=4000)["tflops"]
    gemm_tflops = FLOP_GEMM / (gemm_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": world * FLOP_STEP / (ms_step * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4 (e2m1 x e2m1, ue4m3 group-16 scales), fp32 accumulate", "data": "synthetic",
        "config": {
            "workload": f"NVFP4 W4A4+LoRA linear M={M} K={K} N={N} R={R} (FLUX single-block fused input projection)",
            "per_gpu_rows": M, "l2": "working set per step (28 MB in, 41 MB weights+codes, 198 MB out) exceeds the 126 MB L2",
            "sharding": "rows (M) per rank, no data-path collective",
        },
        "roofline": {
            "kernel": "gemm_w4a4_kernel<NVFP4>", "bound": "tensor", "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s",
            "frac": gemm_tflops / fp4_peak, "traffic": GEMM_DRAM_TRAFFIC if (M, K, N) == (4608, 3072, 21504) else None,
            "traffic_unit": "bytes per launch (dram read + write, one ncu capture of this workload)",
            "peak_source": "measured live: operand-resident tcgen05.mma kind::mxf4nvf4 M128 N256 K64 loop on all SMs "
                           "(burst; MEASURED_PEAKS.json has no FP4 entry); nominal dense FP4 is 9000",
            "frac_of_4x_bf16_measured": gemm_tflops / (4.0 * peaks["bf16_tflops"]), "bf16_peak_kind": peak_kind,
            "avg_launch_us": gemm_ms * 1e3, "launches_timed": len(ev),
            "quantizer": {"bound": "hbm", "achieved": QUANT_BYTES / (quant_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                          "unit": "GB/s", "frac": QUANT_BYTES / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "avg_launch_us": quant_ms * 1e3},
        },
        "e2e": {"value": world * FLOP_STEP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": xh[0].numel() * 2,
                "d2h_bytes_per_step": oh[0].numel() * 2, "ms_per_step": e2e_ms},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        lin, wdeq = cpu_oracle_setup(m)
        rows = 576
        xc = x[:rows].cpu()
        cpu_oracle_step(lin, wdeq, xc[:64])
        t0 = time.perf_counter(); reps = 0
        while reps < 3 or time.perf_counter() - t0 < 10.0:
            cpu_oracle_step(lin, wdeq, xc); reps += 1
            if time.perf_counter() - t0 > 30.0:
                break
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {
            "value": FLOP_STEP * rows / M / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{rows} of {M} rows x {reps} reps (quantise + fp32 dequant-matmul + epilogue; weights kept dequantised)"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
