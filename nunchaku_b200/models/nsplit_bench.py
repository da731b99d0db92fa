"""Time of the N-split variant on a single image: the FLUX single-block fused input projection (M=4608 tokens,
K=3072, N=21504) with the output columns split over the ranks and the bf16 result all-gathered with NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port P \
        -m nunchaku_b200.models.nsplit_bench [--tokens 4608] [--k 3072] [--n 21504] [--precision nvfp4] [--steps 20]

Every rank builds the same random packed weights (same seed), keeps its column shard, quantises the replicated
activations itself and runs the GEMM on its columns; the all-gather puts the ``[M, N]`` result on every rank.  Rank 0
checks the gathered result bit for bit against the unsplit linear, then prints one JSON line: time per call of
quantiser + GEMM + all-gather (CUDA events, max over ranks), of the local part alone, and of the unsplit linear.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _lib
from ..distributed import ColumnParallelW4A4Linear, barrier, init_from_env, max_over_ranks, shutdown
from .mlp_bench import random_linear, timed


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4608)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--n", type=int, default=21504)
    ap.add_argument("--rank", type=int, default=32)
    ap.add_argument("--precision", default="nvfp4", choices=["nvfp4", "int4"])
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    rank, world, local = init_from_env()
    torch.cuda.set_device(local)
    M, K, N = args.tokens, args.k, args.n
    full = random_linear(K, N, args.rank, args.precision, 1)
    par = ColumnParallelW4A4Linear(full, world, rank)
    x = torch.randn(1, M, K, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(0))

    y_full = full(x)
    y = par(x)
    torch.cuda.synchronize()
    equal = bool(torch.equal(y, y_full))
    barrier()
    t_split = max_over_ranks(timed(lambda: par(x), args.steps), "cuda")
    barrier()
    t_local = max_over_ranks(timed(lambda: par.local(x), args.steps), "cuda")
    barrier()
    t_full = max_over_ranks(timed(lambda: full(x), args.steps), "cuda")
    assert _lib.device_status() == (0, 0)
    if rank == 0:
        flop = 2.0 * M * N * K + 2.0 * M * N * args.rank
        print(json.dumps({
            "n_gpus": world, "tokens": M, "K": K, "N": N, "precision": args.precision, "bit_exact_vs_unsplit": equal,
            "nsplit_us": round(t_split, 1), "local_quant_gemm_us": round(t_local, 1), "unsplit_us": round(t_full, 1),
            "nsplit_tflops": round(flop / t_split / 1e6, 1), "allgather_bytes_per_rank": 2 * M * N,
        }))
    shutdown()
    if not equal:
        raise SystemExit("N-split result differs from the unsplit linear")


if __name__ == "__main__":
    main()
