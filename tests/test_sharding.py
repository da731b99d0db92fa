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


# ------------------------------------------------------------------------------------------------ N-split variant
def test_column_shards_partition_columns():
    from nunchaku_b200.distributed import column_shard

    for total in (128, 384, 3072, 21504, 2304):
        for world in (1, 2, 3, 4, 8):
            spans = [column_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a % 128 == 0 and b % 128 == 0
    import pytest

    with pytest.raises(ValueError):
        column_shard(200, 2, 0)


def test_column_shard_of_packed_parameters_is_the_logical_slice():
    """Slicing the reference-packed tensors by byte range gives the packed form of the logical column slice."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import helpers as H
    from oracle import layouts as L
    from oracle import svdq_ref as R
    from nunchaku_b200.distributed import column_shard, shard_linear_columns

    K, N = 256, 640
    for fp4 in (True, False):
        x = R.make_activations(300, K, seed=3)
        lin = R.make_linear(K, N, 32, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=4, wcscales=fp4)
        full = H.to_module(lin, "cpu")
        for world in (2, 5):
            for rank in range(world):
                n0, n1 = column_shard(N, world, rank)
                sh = shard_linear_columns(full, world, rank)
                assert torch.equal(L.ref_unpack_wgt_codes(sh.qweight.view(torch.uint8), K), lin.wcodes[n0:n1])
                assert torch.equal(L.ref_unpack_lora_up(sh.proj_up), lin.lora_up[n0:n1])
                assert torch.equal(L.ref_unpack_vector(sh.bias), lin.bias[n0:n1])
                if fp4:
                    assert torch.equal(L.ref_unpack_wmscales(sh.wscales.view(torch.uint8)), lin.wscales[:, n0:n1])
                    assert torch.equal(L.ref_unpack_vector(sh.wcscales), lin.wcscales[n0:n1])
                    assert torch.equal(sh.wtscale, full.wtscale)
                else:
                    assert torch.equal(L.ref_unpack_wscales(sh.wscales), lin.wscales[:, n0:n1])
                assert torch.equal(sh.proj_down, full.proj_down) and torch.equal(sh.smooth_factor, full.smooth_factor)


def _col_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    from nunchaku_b200.distributed import column_shard, gather_columns

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    for N in (512, 384):   # even and ragged split
        full = torch.arange(37 * N, dtype=torch.float32).view(37, N)
        n0, n1 = column_shard(N, world, rank)
        ok = ok and torch.equal(gather_columns(full[:, n0:n1].contiguous(), N), full)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_two_gloo_ranks_gather_columns():
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 31500 + os.getpid() % 2000
    mp.spawn(_col_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] is True and ret[1] is True
