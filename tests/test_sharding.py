"""Multi-rank host logic on CPU: the row shards cover M exactly, and two gloo ranks that each run the
path on their shard reproduce the single-rank result (the path has no data-path collective)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nunchaku_b200.distributed import gather_rows, max_over_ranks, row_shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_shards_partition_rows():
    for total in (1, 255, 256, 4608, 4609, 36864, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [row_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b and c <= d
            assert all(a % 256 == 0 or a == total for a, _ in spans)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    from oracle import svdq_ref as R

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, K, N = 700, 256, 128
    x = R.make_activations(M, K, seed=0)
    lin = R.make_linear(K, N, 32, fp4=True, x_absmax=x.float().abs().amax(0), seed=1)
    s, e = row_shard(M, world, rank)
    q = R.ref_quantize(x[s:e], lin.smooth, lin.lora_down, fp4=True)
    y_local = R.ref_gemm(q, lin, M=e - s)
    y = gather_rows(y_local, M)
    t = max_over_ranks(float(rank + 1))
    if rank == 0:
        q_full = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=True)
        ret["equal"] = bool(torch.equal(y, R.ref_gemm(q_full, lin, M=M)))
        ret["tmax"] = t
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_single_rank():
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["equal"] is True
    assert ret["tmax"] == 2.0
