#!/usr/bin/env python
"""Benchmark of the SVDQuant W4A4 linear hot path (quantise + 4-bit GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the NVFP4 FLUX single-block fused input projection, M=4608 tokens, K=3072, N=21504,
rank-32 low-rank branch, bf16 in / bf16 out, seeded synthetic data with the value distributions
of the benchmark description (N(0,1) activations with 1% outlier channels x20, N(0,0.02)
weights with the rank-32 SVD component removed, N(0,0.02) low-rank factors and bias).
One step = one pass of the path over one batch: activation quantiser + GEMM.  At N > 1 every rank
runs the same step on its own batch (the path shards along M without communication): weak scaling.
After that leg the same process times, into sub-objects of the same JSON line: the INT4 variant on the M=4096,
K=N=3072 case (`int4_config0`), the FLUX MLP chain (`mlp_chain_config2`), the row-wise kernels and the softmax attention of a
FLUX block (`rowwise_kernels`, `attention`), a FLUX.1-dev-architecture transformer step at global batch 8 (`flux_step`) and a
SANA-1.6B-architecture step at global batch 32 (`sana_step`), both sharded along the batch over the ranks.
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


# dram__bytes_read.sum + dram__bytes_write.sum of one full-size gemm_w4a4_kernel (NVFP4) launch (49.2 MB + 146.2 MB)
GEMM_DRAM_TRAFFIC = 49225472 + 146244608


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


def workload_config():
    return {
        "workload": f"NVFP4 W4A4+LoRA linear M={M} K={K} N={N} R={R} (FLUX single-block fused input projection)",
        "per_gpu_rows": M, "l2": "working set per step (28 MB in, 41 MB weights+codes, 198 MB out) exceeds the 126 MB L2",
        "sharding": "rows (M) per rank, no data-path collective",
    }


DTYPE = "fp4 (e2m1 x e2m1, ue4m3 group-16 scales), fp32 accumulate"


def run_reference(args, rank):
    """Reference arm: the CPU restatement of the reference's arithmetic (the reference has no CPU
    implementation and its NVFP4 kernels have no sm_100 path), all host threads, bounded sample per step."""
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
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": workload_config(),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def event_times(fn_list, reps):
    """Average device time (ms) of each callable in ``fn_list`` run back to back ``reps`` times, one CUDA event between
    every two launches (on torch's current stream, where the library launches).  ``reps`` launches are enqueued while the
    stream is still busy with a delay kernel."""
    n = len(fn_list)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n + 1)] for _ in range(reps)]
    # The stream first gets some milliseconds of idle spinning, so that the host is many launches ahead when the timed kernels
    # start: an interval between two events then never contains a wait for the next launch (on a busy host the enqueue of
    # one pass, with its events, can take longer than the quantiser runs).
    torch.cuda._sleep(int(2.5e7))
    for r in range(reps):
        ev[r][0].record()
        for i, fn in enumerate(fn_list):
            fn()
            ev[r][i + 1].record()
    torch.cuda.synchronize()
    return [sum(ev[r][i].elapsed_time(ev[r][i + 1]) for r in range(reps)) / reps for i in range(n)]


def int4_config0(dev, peaks):
    """The INT4 group-64 variant on the reference's own CPU-runnable case (M=4096, K=N=3072, rank 32): quantiser and GEMM
    times by CUDA events over 50 launches, as absolute TFLOP/s and against the measured tensor-pipe rates of the MMA kind
    the kernel uses (kind::f16, CTA pair) and of the integer kind (kind::i8)."""
    from nunchaku_b200.models.random_init import random_w4a4_linear
    from nunchaku_b200.peak_probe import mma_rate, mma_rate_pair

    M0, K0, N0 = 4096, 3072, 3072
    g = torch.Generator(device=dev).manual_seed(7)
    m = random_w4a4_linear(K0, N0, R, "int4", True, g, dev)
    x = torch.randn(M0, K0, generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty(M0, N0, dtype=torch.bfloat16, device=dev)
    st = {}

    def q():
        st["q"] = m.quantize(x)

    def gm():
        m.forward_quant(*st["q"], out)

    for _ in range(3):
        q(); gm()
    tq, tg = event_times([q, gm], 50)
    flop = 2.0 * M0 * N0 * K0 + 2.0 * M0 * N0 * R
    tf = flop / (tg * 1e-3) / 1e12
    f16 = mma_rate_pair("f16", 256, iters=2000)["tflops"]
    i8 = mma_rate("i8", 256, iters=2000)["tflops"]
    qbytes = 2 * M0 * K0 + M0 * K0 // 2 + M0 * (K0 // 64) * 2 + 4 * M0 * R + 2 * K0 * R + 2 * K0
    return {"workload": f"INT4 W4A4+LoRA linear M={M0} K={K0} N={N0} R={R}", "gemm_us": tg * 1e3, "gemm_tflops": tf,
            "frac_of_f16_pair_mma_rate": tf / f16, "f16_pair_mma_tflops": f16, "frac_of_i8_mma_rate": tf / i8, "i8_mma_tflops": i8,
            "frac_of_bf16_measured": tf / peaks["bf16_tflops"], "quantizer_us": tq * 1e3,
            "quantizer_gbs": qbytes / (tq * 1e-3) / 1e9, "quantizer_frac_hbm": qbytes / (tq * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "launches_timed": 50}


def mlp_chain_config2(dev, peaks, fp4_peak, reps=30):
    """The FLUX MLP chain (M=4608, 3072 -> 12288 with GELU + next-layer requantisation + LoRA-down fused into fc1's GEMM,
    then 12288 -> 3072), rank 32, NVFP4, random packed weights: time of the whole chain and of fc1 / fc2 as plain GEMMs."""
    from nunchaku_b200.models.random_init import random_w4a4_linear
    from nunchaku_b200.ops import fused_gelu_mlp

    Mm, Hd = 4608, 3072
    g = torch.Generator(device=dev).manual_seed(11)
    fc1 = random_w4a4_linear(Hd, 4 * Hd, R, "nvfp4", True, g, dev, bias_std=0.02)
    fc2 = random_w4a4_linear(4 * Hd, Hd, R, "nvfp4", True, g, dev, bias_std=0.02)
    x = torch.randn(1, Mm, Hd, generator=g, device=dev).to(torch.bfloat16)
    for _ in range(3):
        fused_gelu_mlp(x, fc1, fc2)
    chain = event_times([lambda: fused_gelu_mlp(x, fc1, fc2)], reps)[0]
    q1 = fc1.quantize(x.view(Mm, Hd))
    o1 = torch.empty(Mm, 4 * Hd, dtype=torch.bfloat16, device=dev)
    fc1.forward_quant(*q1, o1)
    t1 = event_times([lambda: fc1.forward_quant(*q1, o1)], reps)[0]
    q2 = fc2.quantize(o1)
    o2 = torch.empty(Mm, Hd, dtype=torch.bfloat16, device=dev)
    fc2.forward_quant(*q2, o2)
    t2 = event_times([lambda: fc2.forward_quant(*q2, o2)], reps)[0]
    tq = event_times([lambda: fc1.quantize(x.view(Mm, Hd))], reps)[0]
    flop = 2.0 * Mm * Hd * 4 * Hd * 2 + 2.0 * Mm * R * 5 * Hd
    return {"workload": f"FLUX MLP chain M={Mm}, {Hd} -> {4 * Hd} (GELU + NVFP4 requantisation + LoRA-down in the epilogue) -> {Hd}, R={R}",
            "chain_us": chain * 1e3, "chain_tflops": flop / (chain * 1e-3) / 1e12, "chain_frac_of_fp4_peak": flop / (chain * 1e-3) / 1e12 / fp4_peak,
            "quantizer_us": tq * 1e3, "fc1_plain_gemm_us": t1 * 1e3, "fc2_plain_gemm_us": t2 * 1e3,
            "fc1_requant_gemm_us_est": (chain - tq - t2) * 1e3, "launches_timed": reps}


def rowwise_kernels(dev, peaks, reps=20):
    """The row-wise kernels either side of the W4A4 linears against their algorithmic HBM bytes: RMSNorm + RoPE on a FLUX QKV
    output [4608, 9216], LayerNorm + modulation and the gated residual on [4608, 3072], ReLU linear attention on a SANA QKV output
    [4, 1024, 6912]; and the FLUX QKV projection (3072 -> 9216, NVFP4) with RMSNorm + RoPE inside the GEMM's epilogue against the
    plain projection followed by the row-wise kernel."""
    from nunchaku_b200.models.random_init import random_w4a4_linear
    from nunchaku_b200.ops import gate_residual, layernorm_modulate, litela_attention, qk_norm_rope, qkv_proj_norm_rope

    g = torch.Generator(device=dev).manual_seed(0)
    bf = dict(device=dev, dtype=torch.bfloat16)
    res = {}

    def add(name, fn, byt, shape):
        for _ in range(3):
            fn()
        us = event_times([fn], reps)[0] * 1e3
        res[name] = {"us": us, "GBps": byt / us / 1e3, "frac_hbm": byt / us / 1e3 / peaks["hbm_gbs"], "shape": shape}

    S, heads = 4608, 24
    qkv = torch.randn(1, S, 3 * heads * 128, generator=g, **bf)
    w = torch.ones(128, **bf)
    ang = torch.rand(S, 64, device=dev, generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    add("qk_norm_rope", lambda: qk_norm_rope(qkv, w, w, cos, sin, heads), S * (8 * heads * 128 + 512), [S, 3 * heads * 128])
    x = torch.randn(1, S, 3072, generator=g, **bf)
    sc, sh = torch.randn(1, 3072, generator=g, **bf) * 0.1, torch.randn(1, 3072, generator=g, **bf) * 0.1
    add("layernorm_modulate", lambda: layernorm_modulate(x, sc, sh), S * 3072 * 4, [S, 3072])
    y = torch.randn(1, S, 3072, generator=g, **bf)
    add("gate_residual", lambda: gate_residual(x, sc, y), S * 3072 * 6, [S, 3072])
    proj = random_w4a4_linear(3072, 3 * heads * 128, R, "nvfp4", True, g, dev)
    outs = tuple(torch.empty(1, S, heads * 128, **bf) for _ in range(3))
    for _ in range(3):
        qkv_proj_norm_rope(x, proj, w, w, cos, sin, heads, out=outs)
    t_fused = event_times([lambda: qkv_proj_norm_rope(x, proj, w, w, cos, sin, heads, out=outs)], reps)[0] * 1e3
    t_plain = event_times([lambda: proj(x)], reps)[0] * 1e3
    res["qkv_projection_M4608"] = {"quantise_gemm_with_norm_rope_in_epilogue_us": t_fused, "quantise_gemm_plain_us": t_plain,
                                   "separate_norm_rope_kernel_us": res["qk_norm_rope"]["us"]}
    B, T, lh = 4, 1024, 72
    q = torch.randn(B, T, 3 * lh * 32, generator=g, **bf)
    add("litela_attention", lambda: litela_attention(q, lh), B * T * lh * 32 * 8, [B, T, 3 * lh * 32])
    return res


def attention_kernel(dev, peaks, reps=10, batch=8):
    """The softmax attention of a FLUX block, [batch, 24, 4608, 128] bf16, token-major as the QKV projection's epilogue leaves it:
    this library's tcgen05 kernel against the measured bf16 matmul peak (4 * B * H * T^2 * 128 flop), with torch's library
    attention on the same tensors beside it."""
    from nunchaku_b200.ops import attention

    H_, T, D_ = 24, 4608, 128
    g = torch.Generator(device=dev).manual_seed(3)
    q, k, v = (torch.randn(batch, T, H_, D_, generator=g, device=dev).to(torch.bfloat16).transpose(1, 2) for _ in range(3))
    out = torch.empty(batch, T, H_ * D_, device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        attention(q, k, v, out=out)
        torch.nn.functional.scaled_dot_product_attention(q, k, v)
    t_own = event_times([lambda: attention(q, k, v, out=out)], reps)[0]
    t_lib = event_times([lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v)], reps)[0]
    flop = 4.0 * batch * H_ * T * T * D_
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(batch, T, H_ * D_).float()
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    tf = flop / (t_own * 1e-3) / 1e12
    one = {}
    if batch > 1:   # one image: what a rank runs when the step's batch is sharded over eight GPUs (2.9 waves of CTAs)
        q1, k1, v1 = (torch.randn(1, T, H_, D_, generator=g, device=dev).to(torch.bfloat16).transpose(1, 2) for _ in range(3))
        o1 = torch.empty(1, T, H_ * D_, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            attention(q1, k1, v1, out=o1)
            torch.nn.functional.scaled_dot_product_attention(q1, k1, v1)
        one = {"one_image_us": event_times([lambda: attention(q1, k1, v1, out=o1)], reps)[0] * 1e3,
               "one_image_library_sdpa_us": event_times([lambda: torch.nn.functional.scaled_dot_product_attention(q1, k1, v1)], reps)[0] * 1e3}
    return {**one, "workload": f"softmax attention [{batch}, {H_}, {T}, {D_}] bf16, token-major", "kernel": "attention_fwd_kernel (tcgen05, TMEM)",
            "us": t_own * 1e3, "tflops": tf, "frac_bf16_peak": tf / peaks["bf16_tflops"], "peak_bf16_tflops": peaks["bf16_tflops"],
            "library_sdpa_us": t_lib * 1e3, "library_sdpa_tflops": flop / (t_lib * 1e-3) / 1e12, "rel_l2_vs_library": rel,
            "launches_timed": reps}


def reference_int4_kernels(dev):
    """The reference's own INT4 kernels (compiled from the reference tree into oracle/_ref, mma.sync, no sm_100 tuning)
    timed on this GPU on the same case as ``int4_config0``: a baseline beside the CPU port, not the product path."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import ref_int4 as REF
    if not REF.available():
        return None
    from nunchaku_b200.models.random_init import random_w4a4_linear
    M0, K0, N0 = 4096, 3072, 3072
    g = torch.Generator(device=dev).manual_seed(7)
    m = random_w4a4_linear(K0, N0, R, "int4", True, g, dev)
    x = torch.randn(M0, K0, generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty(M0, N0, dtype=torch.bfloat16, device=dev)
    st = {}

    def q():
        st["q"] = REF.quantize(x, m.smooth_factor, m.proj_down)

    def gm():
        c, s, la = st["q"]
        REF.gemm(c, m.qweight, s, m.wscales, out=out, lora_act_in=la, lora_up=m.proj_up, bias=m.bias)

    for _ in range(3):
        q(); gm()
    tq, tg = event_times([q, gm], 20)
    flop = 2.0 * M0 * N0 * K0 + 2.0 * M0 * N0 * R
    return {"workload": f"INT4 W4A4+LoRA linear M={M0} K={K0} N={N0} R={R}", "kind": "reference kernels (mma.sync s4, "
            "bf16 accumulation) compiled for sm_100a", "gemm_us": tg * 1e3, "gemm_tflops": flop / (tg * 1e-3) / 1e12,
            "quantizer_us": tq * 1e3, "launches_timed": 20}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-model-steps", action="store_true", help="skip the FLUX / SANA transformer-step legs and the INT4 case")
    ap.add_argument("--only", default=None, choices=["mlp", "int4", "rowwise", "attention"],
                    help="profiler captures: run just this leg (a few launches of it) and print its record")
    ap.add_argument("--shape", default=None, help="M,K,N override: a smaller case of the same path for profiler captures "
                    "(the default is the benchmark workload); implies --no-model-steps")
    args = ap.parse_args()
    if args.shape:
        global M, K, N, FLOP_GEMM, FLOP_STEP, QUANT_BYTES
        M, K, N = (int(v) for v in args.shape.split(","))
        FLOP_GEMM = 2.0 * M * N * K + 2.0 * M * N * R
        FLOP_STEP = FLOP_GEMM
        QUANT_BYTES = 2 * M * K + M * K // 2 + M * K // 16 + 4 * M * R + 2 * K * R + 2 * K
        args.no_model_steps = True
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
    if args.only:
        peaks, _ = load_peaks()
        if args.only == "mlp":
            rec = mlp_chain_config2(dev, peaks, 8500.0, reps=max(2, args.steps))
        elif args.only == "rowwise":
            rec = rowwise_kernels(dev, peaks, reps=max(2, args.steps))
        elif args.only == "attention":   # one image: a capture-sized case of the same kernel
            rec = attention_kernel(dev, peaks, reps=max(2, args.steps), batch=1)
        else:
            rec = int4_config0(dev, peaks)
        print(json.dumps(rec), flush=True)
        return

    x = make_inputs(dev, rank)
    m = build_layer(dev, 0, x)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    st = {}

    def quant():
        st["q"] = m.quantize(x)

    def gemm():
        m.forward_quant(*st["q"], out)

    def step():
        quant()
        gemm()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    # ---- timed region: K steps on inputs resident in HBM.  A step is `inner` back-to-back passes of the path (chosen so
    # that the region lasts >= 50 ms: with a 0.17 ms pass and a MAX over ranks, a region of a few ms is set by the one
    # rank whose host hiccuped); ms_per_step is per pass.  No event is recorded inside the region.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        step()
    e1.record()
    torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1) / 3, 1e-3)
    inner = max(1, int(50.0 / (est * args.steps) + 0.999))
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    D.barrier()
    torch.cuda.synchronize()
    # a few milliseconds of idle spinning on the stream in front of the first event: the host is launches ahead when the
    # clock starts, so its start-up latency (eight ranks share one host) is not in the interval
    torch.cuda._sleep(int(1.0e7))
    t_host = time.perf_counter()
    e0.record()
    for _ in range(args.steps * inner):
        step()
    e1.record()
    host_ms = (time.perf_counter() - t_host) * 1e3 / (args.steps * inner)
    torch.cuda.synchronize()
    D.barrier()
    ms_local = e0.elapsed_time(e1) / (args.steps * inner)
    if sampler:   # keep the load up until the sampler has a few samples of it
        t_end = time.time() + 0.5
        while time.time() < t_end:
            for _ in range(50):
                step()
            torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms_step = D.max_over_ranks(ms_local, dev)
    per_rank = {"ms_per_step": {"min": -D.max_over_ranks(-ms_local, dev), "max": ms_step},
                "host_enqueue_ms_per_step": {"min": -D.max_over_ranks(-host_ms, dev), "max": D.max_over_ranks(host_ms, dev)}}
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms_local], dtype=torch.float64, device=dev)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        vals = sorted(float(v.item()) for v in allt)
        per_rank["ms_per_step"]["median"] = vals[len(vals) // 2]
        per_rank["ms_per_step"]["all"] = [round(v, 5) for v in vals]
    # ---- per-kernel durations for the roofline figures: the same passes again with an event between the two kernels,
    # >= 50 launches of each (an event between two kernels keeps the second one's launch from overlapping the first one's
    # tail, which is why the region above carries none)
    launches = max(50, args.steps)
    quant_ms, gemm_ms = event_times([quant, gemm], launches)
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
    e0.record()
    pipe.fork()
    for i in range(e2e_steps):
        pipe.submit(xh[i % 2], oh[i % 2])
    pipe.join()
    e1.record()
    torch.cuda.synchronize()
    if not torch.equal(oh[0], out.cpu()) or not torch.equal(oh[1], oh[0]):
        raise SystemExit("end-to-end result differs from the device-resident result")
    e2e_ms = D.max_over_ranks(e0.elapsed_time(e1) / e2e_steps, dev)
    del pipe, xh, oh

    peaks, peak_kind = load_peaks()
    # FP4 has no entry in MEASURED_PEAKS.json: measure the tensor-pipe peak here, on this GPU, with the
    # library's operand-resident tcgen05.mma loop (kind::mxf4nvf4, M128 N256 K64 per instruction).
    from nunchaku_b200.peak_probe import mma_rate
    probe = mma_rate("mxf4nvf4", 256, iters=4000)
    fp4_peak = probe["tflops"]
    # The probe moves no data and runs near the maximum clock; the GEMM runs under the power cap (clocks.sm_mhz).  The same
    # peak scaled to the clock the GEMM saw says how well the kernel uses the cycles it gets.
    gemm_mhz = clocks["sm_mhz"] if clocks and clocks.get("sm_mhz") else None
    peak_at_gemm_clock = fp4_peak * gemm_mhz / probe["sm_mhz"] if gemm_mhz else None
    gemm_tflops = FLOP_GEMM / (gemm_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": world * FLOP_STEP / (ms_step * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": workload_config(),
        "timed_region": {"passes_per_step": inner, "passes": args.steps * inner, "ms": ms_step * args.steps * inner,
                         "note": "ms_per_step and value are per pass of the path (quantiser + GEMM)"},
        "per_rank": per_rank,
        "roofline": {
            "kernel": "gemm_w4a4_kernel<NVFP4>", "bound": "tensor", "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s",
            "frac": gemm_tflops / fp4_peak, "traffic": GEMM_DRAM_TRAFFIC if (M, K, N) == (4608, 3072, 21504) else None,
            "traffic_unit": "bytes per launch (dram read + write, one ncu capture of this workload)",
            "peak_source": "measured live: operand-resident tcgen05.mma kind::mxf4nvf4 M128 N256 K64 loop on all SMs "
                           "(burst; MEASURED_PEAKS.json has no FP4 entry); nominal dense FP4 is 9000",
            "peak_probe_sm_mhz": probe["sm_mhz"], "peak_at_gemm_clock": peak_at_gemm_clock,
            "frac_at_equal_clock": gemm_tflops / peak_at_gemm_clock if peak_at_gemm_clock else None,
            "frac_of_4x_bf16_measured": gemm_tflops / (4.0 * peaks["bf16_tflops"]), "bf16_peak_kind": peak_kind,
            "avg_launch_us": gemm_ms * 1e3, "launches_timed": launches,
            "quantizer": {"bound": "hbm", "achieved": QUANT_BYTES / (quant_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                          "unit": "GB/s", "frac": QUANT_BYTES / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "avg_launch_us": quant_ms * 1e3, "launches_timed": launches},
        },
        "e2e": {"value": world * FLOP_STEP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_ms,
                "note": "bound by the copy of the bf16 result to the host (PCIe); all ranks share one host memory complex. "
                        "A consumer that is another W4A4 layer takes the requantised 4-bit output instead (4x fewer bytes)"},
        "gpu_launches": 2 * args.steps * inner,
        "clocks": clocks,
    }
    del out, x
    if not args.no_model_steps:
        torch.cuda.empty_cache()
        if rank == 0:
            line["int4_config0"] = int4_config0(dev, peaks)
            line["mlp_chain_config2"] = mlp_chain_config2(dev, peaks, fp4_peak)
            line["rowwise_kernels"] = rowwise_kernels(dev, peaks)
            line["attention"] = attention_kernel(dev, peaks)
        D.barrier()
        from nunchaku_b200.models import flux_bench, sana_bench
        line["flux_step"] = flux_bench.run(global_batch=8, reps=10, warmup=2, graph=True)
        torch.cuda.empty_cache()
        line["sana_step"] = sana_bench.run(global_batch=32, reps=10, warmup=2, graph=True)
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        lin, wdeq = cpu_oracle_setup(m)
        rows = 576
        xc = make_inputs(dev, rank)[:rows].cpu()
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
        if not args.no_model_steps:
            try:
                line["reference_int4_kernels"] = reference_int4_kernels(dev)
            except Exception as exc:   # a baseline beside the port: never fail the benchmark over it
                line["reference_int4_kernels"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    D.shutdown()


if __name__ == "__main__":
    main()
