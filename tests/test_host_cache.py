"""Host-side caches of the GEMM wrapper must not outlive the tensors they were built from."""
import numpy as np
import torch

from nunchaku_b200.ops import gemm as G


def test_alpha_cache_is_not_fooled_by_a_recycled_address():
    buf = np.array([2.0], dtype=np.float32)
    t1 = torch.from_numpy(buf)
    assert G._alpha_value(t1) == 2.0
    assert G._alpha_value(t1) == 2.0          # served from the cache
    key = G._ident(t1)
    del t1
    buf[0] = 3.0                              # "freed and reallocated": same address, version and shape
    t2 = torch.from_numpy(buf)
    assert G._ident(t2) == key
    assert G._alpha_value(t2) == 3.0


def test_alpha_cache_follows_in_place_updates():
    t = torch.tensor([1.5])
    assert G._alpha_value(t) == 1.5
    t.fill_(0.25)                             # bumps the version counter
    assert G._alpha_value(t) == 0.25
    assert G._alpha_value(None) == 1.0 and G._alpha_value(0.5) == 0.5
