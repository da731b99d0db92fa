"""N-split variant on the GPU: the column shards of a W4A4 linear, run one after the other on one GPU, reproduce the
unsplit linear bit for bit (every output element sees the same operands in the same k order whichever tile holds
it), in both precisions and with a ragged split."""
import pytest
import torch

import helpers as H
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fp4", [True, False])
@pytest.mark.parametrize("world", [2, 3])
def test_column_shards_reproduce_the_full_linear(fp4, world):
    from nunchaku_b200 import _lib
    from nunchaku_b200.distributed import column_shard, shard_linear_columns

    M, K, N = 520, 512, 1152
    x = R.make_activations(M, K, seed=5)
    lin = R.make_linear(K, N, 32, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=6, mode="svd", wcscales=fp4)
    full = H.to_module(lin, "cuda:0")
    xg = x.cuda().view(1, M, K)
    y = full(xg).view(M, N)
    parts = []
    for rank in range(world):
        n0, n1 = column_shard(N, world, rank)
        yr = shard_linear_columns(full, world, rank)(xg).view(M, n1 - n0)
        parts.append(yr)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.equal(torch.cat(parts, dim=1), y)
    q = R.ref_quantize(x, lin.smooth, lin.lora_down, fp4=fp4)
    assert R.rel_l2(y.float().cpu(), R.ref_gemm(q, lin, M=M)) <= 1e-2   # tolerance of the path: relative L2 <= 1e-2
