"""HostPipeline: three-stream, double-buffered host -> device -> host path gives the same bits as direct calls."""
import pytest
import torch

import helpers as H
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_direct_calls():
    from nunchaku_b200.host_pipeline import HostPipeline

    M, K, N = 512, 256, 384
    xs = [R.make_activations(M, K, seed=40 + i) for i in range(5)]
    lin = R.make_linear(K, N, 32, fp4=True, x_absmax=xs[0].float().abs().amax(0), seed=9, mode="svd")
    m = H.to_module(lin)
    direct = [m(x.cuda().view(1, M, K)).view(M, N).cpu() for x in xs]
    xh = [x.view(1, M, K).pin_memory() for x in xs]
    oh = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in xs]
    pipe = HostPipeline(m, (1, M, K), (M, N))
    for x, o in zip(xh, oh):
        pipe.submit(x, o)
    pipe.join()
    torch.cuda.synchronize()
    for d, o in zip(direct, oh):
        assert torch.equal(d, o)
