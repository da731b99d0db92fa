"""The W4A4 linear and the fused MLP chain captured in a CUDA graph replay to the eager result bit for bit (after one
warm-up call, which builds the prepared-weight cache, the ops allocate only through torch's capture-aware pool and
never synchronise)."""
import pytest
import torch

import helpers as H
from oracle import svdq_ref as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fp4", [True, False])
def test_linear_and_mlp_chain_in_a_cuda_graph(fp4):
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops import fused_gelu_mlp

    M, K, N = 520, 512, 1024
    x = R.make_activations(M, K, seed=21)
    fc1 = H.to_module(R.make_linear(K, N, 32, fp4=fp4, x_absmax=x.float().abs().amax(0), seed=22, wcscales=fp4), "cuda:0",
                      act_unsigned=False)
    fc2 = H.to_module(R.make_linear(N, K, 32, fp4=fp4, x_absmax=torch.rand(N) + 0.5, seed=23, wcscales=fp4), "cuda:0",
                      act_unsigned=not fp4)
    xg = x.cuda().view(1, M, K)
    with torch.no_grad():
        y_eager, z_eager = fc1(xg).clone(), fused_gelu_mlp(xg, fc1, fc2).clone()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                y = fc1(xg)
                z = fused_gelu_mlp(xg, fc1, fc2)
        for _ in range(2):
            y.zero_()
            z.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(y, y_eager) and torch.equal(z, z_eager)
    assert _lib.device_status() == (0, 0)


def test_attention_in_a_cuda_graph():
    """Captured after one warm-up call (which caches the per-device state), the attention kernel replays to the eager result
    bit for bit: it is deterministic (no atomics) and neither allocates outside torch's pool nor synchronises."""
    from nunchaku_b200 import _lib
    from nunchaku_b200.ops import attention

    g = torch.Generator(device="cuda").manual_seed(9)
    q, k, v = (torch.randn(2, 333, 3, 128, device="cuda", generator=g).bfloat16().transpose(1, 2) for _ in range(3))
    o_eager = attention(q, k, v).clone()
    assert torch.equal(attention(q, k, v), o_eager)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):
            o = attention(q, k, v)
    for _ in range(2):
        o.zero_()
        cg.replay()
        torch.cuda.synchronize()
        assert torch.equal(o, o_eager)
    assert _lib.device_status() == (0, 0)
