"""Step time of a SANA-1.6B-architecture linear DiT whose block linears run on the W4A4 path (INT4 group 64 by default).

    python -m nunchaku_b200.models.sana_bench [--batch 32] [--steps 5] [--precision int4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m nunchaku_b200.models.sana_bench --batch 32

1024 x 1024 pixels = 32 x 32 latent tokens of 32 channels per image, 300 caption tokens; the global batch is sharded along
the batch dimension over the ranks (no data-path collective).  Weights are random packed W4A4 parameters (no checkpoints
offline).  Prints one JSON line on rank 0: image-steps per second over all ranks (time = max over ranks, CUDA events).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _lib
from .. import distributed as D
from .sana import SanaTransformer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32, help="global batch (images per step over all ranks)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--graph", action="store_true", help="capture one forward in a CUDA graph and time its replays "
                    "(small per-GPU batches are bound by launch overhead otherwise)")
    ap.add_argument("--precision", default="int4", choices=["nvfp4", "int4"])
    ap.add_argument("--blocks", type=int, default=20)
    args = ap.parse_args()
    rank, world, local = D.init_from_env()
    torch.cuda.set_device(local)
    if args.batch % world:
        raise SystemExit("--batch must be a multiple of the number of ranks")
    B = args.batch // world
    torch.manual_seed(rank)
    model = SanaTransformer(n_blocks=args.blocks, precision=args.precision, seed=rank)
    H = W = 32
    lat = torch.randn(B, H * W, 32, device="cuda", dtype=torch.bfloat16)
    cap = torch.randn(B, 300, 2304, device="cuda", dtype=torch.bfloat16)
    t = torch.full((B,), 0.5, device="cuda")
    with torch.no_grad():
        for _ in range(args.warmup):
            y = model(lat, cap, t, (H, W))
        graph = None
        if args.graph:
            # every prepared-weight cache and status word exists after the warm-up, so nothing allocates outside torch's
            # capture-aware pool and nothing synchronises inside the captured region
            y_eager = y.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y = model(lat, cap, t, (H, W))
            graph.replay()
            torch.cuda.synchronize()
            if not torch.equal(y, y_eager):
                raise SystemExit("graph replay differs from the eager forward")
        D.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            if graph is not None:
                graph.replay()
            else:
                y = model(lat, cap, t, (H, W))
        e1.record()
        torch.cuda.synchronize()
    ms = D.max_over_ranks(e0.elapsed_time(e1) / args.steps, "cuda")
    finite = bool(torch.isfinite(y).all())
    assert _lib.device_status() == (0, 0)
    if rank == 0:
        print(json.dumps({
            "metric": "SANA-1.6B-architecture 1024px image-steps/s", "value": round(args.batch / ms * 1e3, 2), "ms_per_step": round(ms, 3),
            "n_gpus": world, "global_batch": args.batch, "per_gpu_batch": B, "precision": args.precision, "blocks": args.blocks,
            "w4a4_linears": len(model.w4a4_linears()), "finite": finite, "cuda_graph": bool(args.graph), "weights": "random packed W4A4", "scaling": "strong",
        }))
    D.shutdown()


if __name__ == "__main__":
    main()
