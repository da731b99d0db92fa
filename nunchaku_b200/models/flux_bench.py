"""Step time of a FLUX.1-dev-architecture transformer whose block linears run on the W4A4 path.

    python -m nunchaku_b200.models.flux_bench [--batch 8] [--reps 10] [--precision nvfp4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m nunchaku_b200.models.flux_bench --batch 8

1024 x 1024 pixels = 64 x 64 patchified latent = 4096 image tokens + 512 text tokens per image; the global batch is
sharded along the batch dimension over the ranks (no data-path collective).  The model is random-init bf16 and its 304
block linears are then quantised on the GPU the SVDQuant way (smoothing, rank-32 SVD branch, NVFP4 group-16 residual:
``FluxTransformer.quantize_``); ``--random-packed`` fills packed parameters with random codes instead (faster start).
Attention is torch SDPA, embedders and modulation linears are bf16 ``nn.Linear``.
Prints one JSON line on rank 0: image-steps per second over all ranks (time = max over ranks, CUDA events).
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from .. import _lib
from .. import distributed as D
from . import flux as F_
from .flux import FluxTransformer
from .step_timing import device_time_split, timed_steps


def run(global_batch: int = 8, reps: int = 10, warmup: int = 2, precision: str = "nvfp4", joint: int = 19, single: int = 38,
        graph: bool = False, random_packed: bool = False, split: bool = True) -> dict:
    """Build the model on the current device, time ``reps`` steps of this rank's share of ``global_batch`` and return the
    result record (identical on every rank; times are the maximum over ranks)."""
    rank, world, local = D.init_from_env()
    dev = torch.device("cuda", torch.cuda.current_device())
    if global_batch % world:
        raise ValueError("the global batch must be a multiple of the number of ranks")
    B = global_batch // world
    torch.manual_seed(rank)
    t0 = time.perf_counter()
    model = FluxTransformer(precision=None, n_joint=joint, n_single=single, device=dev)
    if random_packed:
        model.randomize_w4a4_(precision, 32, seed=rank)
    else:
        model.quantize_(precision, 32)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    H = W = 64
    T = 512
    lat = torch.randn(B, H * W, 64, device=dev, dtype=torch.bfloat16)
    txt = torch.randn(B, T, 4096, device=dev, dtype=torch.bfloat16)
    pooled = torch.randn(B, 768, device=dev, dtype=torch.bfloat16)
    t = torch.full((B,), 0.5, device=dev)
    g = torch.full((B,), 3.5, device=dev)
    out = {}

    def eager():
        out["y"] = model(lat, txt, pooled, t, g, (H, W))

    with torch.no_grad():
        step = eager
        graph_note = None
        if graph:
            try:
                # every prepared-weight copy and per-device cache exists after the warm-up, so nothing allocates outside torch's
                # capture-aware pool and nothing synchronises inside the captured region
                for _ in range(2):
                    eager()
                y_eager = out["y"].clone()
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg):
                    eager()
                cg.replay()
                torch.cuda.synchronize()
                if not torch.equal(out["y"], y_eager):
                    raise RuntimeError("graph replay differs from the eager forward")
                step = cg.replay
            except Exception as exc:   # capture is an optimisation of the host side only: fall back to eager launches
                step, graph, graph_note = eager, False, f"{type(exc).__name__}: {exc}"[:160]
                torch.cuda.synchronize()
        D.barrier()
        t_host = time.perf_counter()
        host = {}
        ms, per_run = timed_steps(step, reps, warmup, host)
        wall_ms = (time.perf_counter() - t_host) * 1e3 / (reps + warmup)
        prof = device_time_split(eager) if (split and rank == 0) else None
        # the same step with the library's attention in place of this library's kernel, both by eager launches
        compare = {}
        if split:
            for name in ("tcgen05", "sdpa"):
                F_.ATTENTION_BACKEND["name"] = name
                compare[name + "_ms"] = round(D.max_over_ranks(timed_steps(eager, 3, 1, {})[0], dev), 2)
            F_.ATTENTION_BACKEND["name"] = "tcgen05"
            compare["mode"] = "eager launches, 3 runs each, max over ranks"
    ms_max = D.max_over_ranks(ms, dev)
    ms_min = -D.max_over_ranks(-ms, dev)
    status = _lib.device_status()
    if status != (0, 0):
        raise RuntimeError(f"device status {status}: a bounded wait ran out")
    return {
        "workload": f"FLUX.1-dev-architecture transformer step, 1024x1024 (4096 image + {T} text tokens), {joint} joint + "
                    f"{single} single blocks, {precision} W4A4 linears, global batch {global_batch}",
        "image_steps_per_s": global_batch / (ms_max * 1e-3), "ms_per_step": ms_max, "ms_per_step_min_rank": ms_min,
        "per_gpu_batch": B, "global_batch": global_batch, "n_gpus": world, "scaling": "strong", "speedup_basis": "image_steps_per_s", "reps": reps, "warmup": warmup,
        "protocol": "2 warm-ups, timed runs with CUDA events, fastest and slowest 20 % dropped, max over ranks",
        "w4a4_linears": len(model.w4a4_linears()), "weights": "random packed" if random_packed else "random-init bf16, quantised on the GPU (smooth, rank-32 SVD, group quantise)",
        "model_build_s": round(build_s, 1), "host_ms_per_step": round(wall_ms, 2), "host_enqueue_ms_per_step": round(host.get("enqueue_ms_per_step", 0.0), 2), "cuda_graph": bool(graph), "cuda_graph_fallback": graph_note,
        "finite": bool(torch.isfinite(out["y"]).all()), "device_time_split": prof, "per_run_ms": [round(v, 2) for v in per_run],
        "attention_compare": compare,
        "attention": ("svdq_attention (this library's tcgen05 kernel, csrc/attention.cu)" if F_.ATTENTION_BACKEND["name"] == "tcgen05"
                      else "torch scaled_dot_product_attention (library kernel)"),
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8, help="global batch (images per step over all ranks)")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--graph", action="store_true", help="capture one forward in a CUDA graph and time its replays")
    ap.add_argument("--random-packed", action="store_true", help="random packed parameters instead of quantising bf16 weights")
    ap.add_argument("--precision", default="nvfp4", choices=["nvfp4", "int4"])
    ap.add_argument("--joint", type=int, default=19)
    ap.add_argument("--single", type=int, default=38)
    args = ap.parse_args()
    rank, world, local = D.init_from_env()
    torch.cuda.set_device(local)
    rec = run(args.batch, args.reps, args.warmup, args.precision, args.joint, args.single, args.graph, args.random_packed)
    if rank == 0:
        print(json.dumps(rec))
    D.barrier()
    D.shutdown()


if __name__ == "__main__":
    main()
