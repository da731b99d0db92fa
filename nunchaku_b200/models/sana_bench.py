"""Step time of a SANA-1.6B-architecture linear DiT whose block linears run on the W4A4 path (INT4 group 64).

    python -m nunchaku_b200.models.sana_bench [--batch 32] [--reps 10]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m nunchaku_b200.models.sana_bench --batch 32

1024 px = 32 x 32 latent tokens of 32 channels, 300 caption tokens; the global batch is sharded along the batch dimension
over the ranks (no data-path collective).  Weights are random packed W4A4 parameters (no checkpoints offline).
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from .. import _lib
from .. import distributed as D
from .sana import SanaTransformer
from .step_timing import device_time_split, timed_steps


def run(global_batch: int = 32, reps: int = 10, warmup: int = 2, precision: str = "int4", blocks: int = 20, graph: bool = False,
        split: bool = True) -> dict:
    rank, world, local = D.init_from_env()
    dev = torch.device("cuda", torch.cuda.current_device())
    if global_batch % world:
        raise ValueError("the global batch must be a multiple of the number of ranks")
    B = global_batch // world
    torch.manual_seed(rank)
    model = SanaTransformer(n_blocks=blocks, precision=precision, seed=rank, device=dev)
    H = W = 32
    lat = torch.randn(B, H * W, 32, device=dev, dtype=torch.bfloat16)
    cap = torch.randn(B, 300, 2304, device=dev, dtype=torch.bfloat16)
    t = torch.full((B,), 0.5, device=dev)
    out = {}

    def eager():
        out["y"] = model(lat, cap, t, (H, W))

    with torch.no_grad():
        step = eager
        graph_note = None
        if graph:
            try:
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
    ms_max = D.max_over_ranks(ms, dev)
    ms_min = -D.max_over_ranks(-ms, dev)
    status = _lib.device_status()
    if status != (0, 0):
        raise RuntimeError(f"device status {status}: a bounded wait ran out")
    return {
        "workload": f"SANA-1.6B-architecture linear DiT step, 1024px (1024 tokens), {blocks} blocks, {precision} W4A4 linears, "
                    f"global batch {global_batch}",
        "image_steps_per_s": global_batch / (ms_max * 1e-3), "ms_per_step": ms_max, "ms_per_step_min_rank": ms_min,
        "per_gpu_batch": B, "global_batch": global_batch, "n_gpus": world, "scaling": "strong", "speedup_basis": "image_steps_per_s", "reps": reps, "warmup": warmup,
        "protocol": "2 warm-ups, timed runs with CUDA events, fastest and slowest 20 % dropped, max over ranks",
        "w4a4_linears": len(model.w4a4_linears()), "weights": "random packed W4A4", "host_ms_per_step": round(wall_ms, 2), "host_enqueue_ms_per_step": round(host.get("enqueue_ms_per_step", 0.0), 2),
        "cuda_graph": bool(graph), "cuda_graph_fallback": graph_note, "finite": bool(torch.isfinite(out["y"]).all()), "device_time_split": prof,
        "per_run_ms": [round(v, 2) for v in per_run],
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32, help="global batch (images per step over all ranks)")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--graph", action="store_true", help="capture one forward in a CUDA graph and time its replays")
    ap.add_argument("--precision", default="int4", choices=["nvfp4", "int4"])
    ap.add_argument("--blocks", type=int, default=20)
    args = ap.parse_args()
    rank, world, local = D.init_from_env()
    torch.cuda.set_device(local)
    rec = run(args.batch, args.reps, args.warmup, args.precision, args.blocks, args.graph)
    if rank == 0:
        print(json.dumps(rec))
    D.barrier()
    D.shutdown()


if __name__ == "__main__":
    main()
