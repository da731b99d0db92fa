"""Step time of a FLUX.1-dev-architecture transformer whose block linears run on the W4A4 path.

    python -m nunchaku_b200.models.flux_bench [--batch 8] [--steps 5] [--precision nvfp4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m nunchaku_b200.models.flux_bench --batch 8

1024 x 1024 pixels = 64 x 64 patchified latent = 4096 image tokens + 512 text tokens per image; the global batch is
sharded along the batch dimension over the ranks (no data-path collective).  Weights are random: the block linears get
random packed W4A4 parameters (``FluxTransformer.randomize_w4a4_``), since quantising 12 B master weights on the CPU
takes hours and there are no checkpoints offline.  Attention is torch SDPA, embedders and modulation linears are bf16
``nn.Linear``; RMSNorm + RoPE of q/k and LayerNorm + modulation run as the library's row-wise kernels.
Prints one JSON line on rank 0: image-steps per second over all ranks (time = max over ranks, CUDA events).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _lib
from .. import distributed as D
from .flux import FluxTransformer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8, help="global batch (images per step over all ranks)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--graph", action="store_true", help="capture one forward in a CUDA graph and time its replays "
                    "(small per-GPU batches are bound by launch overhead otherwise)")
    ap.add_argument("--precision", default="nvfp4", choices=["nvfp4", "int4"])
    ap.add_argument("--joint", type=int, default=19)
    ap.add_argument("--single", type=int, default=38)
    args = ap.parse_args()
    rank, world, local = D.init_from_env()
    torch.cuda.set_device(local)
    if args.batch % world:
        raise SystemExit("--batch must be a multiple of the number of ranks")
    B = args.batch // world
    torch.manual_seed(rank)
    model = FluxTransformer(precision=None, n_joint=args.joint, n_single=args.single)
    model.randomize_w4a4_(args.precision, 32, seed=rank)
    H = W = 64
    T = 512
    lat = torch.randn(B, H * W, 64, device="cuda", dtype=torch.bfloat16)
    txt = torch.randn(B, T, 4096, device="cuda", dtype=torch.bfloat16)
    pooled = torch.randn(B, 768, device="cuda", dtype=torch.bfloat16)
    t = torch.full((B,), 0.5, device="cuda")
    g = torch.full((B,), 3.5, device="cuda")
    with torch.no_grad():
        for _ in range(args.warmup):
            y = model(lat, txt, pooled, t, g, (H, W))
        graph = None
        if args.graph:
            # every prepared-weight cache and status word exists after the warm-up, so nothing allocates outside torch's
            # capture-aware pool and nothing synchronises inside the captured region
            y_eager = y.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y = model(lat, txt, pooled, t, g, (H, W))
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
                y = model(lat, txt, pooled, t, g, (H, W))
        e1.record()
        torch.cuda.synchronize()
    ms = D.max_over_ranks(e0.elapsed_time(e1) / args.steps, torch.device("cuda", local))
    status = _lib.device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "FLUX-architecture 1024px transformer, image-steps per second", "value": args.batch / (ms * 1e-3),
            "unit": "image-steps/s", "n_gpus": world, "ms_per_step": ms, "global_batch": args.batch, "per_gpu_batch": B,
            "precision": args.precision, "blocks": [args.joint, args.single], "tokens_per_image": H * W + T,
            "w4a4_linears": len(model.w4a4_linears()), "data": "synthetic, random packed weights",
            "finite": bool(torch.isfinite(y).all()), "cuda_graph": bool(args.graph), "device_status": list(status),
        }))
    D.barrier()
    D.shutdown()


if __name__ == "__main__":
    main()
