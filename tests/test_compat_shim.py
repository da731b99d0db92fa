"""``nunchaku_b200._C`` stands in for the reference's compiled ``nunchaku._C`` on the W4A4 path.

CPU part (needs the reference tree, skipped where it is absent): the reference's OWN ``nunchaku/ops/quantize.py``,
``gemm.py``, ``fused.py`` and ``nunchaku/models/linear.py`` are loaded by file path with ``nunchaku._C`` bound to the shim;
a recorder in place of the two ops checks that what those files pass binds to the shim's positional signatures and
arrives with the reference's meaning.  GPU part: the same calling pattern (caller-allocated outputs, 8 and 29
positional arguments) runs through the shim and matches this package's own module.
"""
import importlib.util
import inspect
import os
import sys
import types
from pathlib import Path

import pytest
import torch

REF = Path(os.environ.get("NUNCHAKU_REFERENCE", "/root/reference"))

GEMM_ARGS = ["act", "wgt", "out", "qout", "ascales", "wscales", "oscales", "poolout", "lora_act_in", "lora_up", "lora_down",
             "lora_act_out", "norm_q", "norm_k", "rotary_emb", "bias", "smooth_factor", "out_vk", "out_linearattn",
             "act_unsigned", "lora_scales", "fuse_silu", "fp4", "alpha", "wcscales", "out_q", "out_k", "out_v", "attn_tokens"]
QUANT_ARGS = ["input", "output", "oscales", "lora_down", "lora_act_out", "smooth", "fuse_glu", "fp4"]


def test_shim_signatures_follow_the_reference_binding():
    from nunchaku_b200 import _C

    assert list(inspect.signature(_C.ops.gemm_w4a4).parameters) == GEMM_ARGS            # nunchaku/csrc/ops.h:10-38
    assert list(inspect.signature(_C.ops.quantize_w4a4_act_fuse_lora).parameters) == QUANT_ARGS   # ops.h:82-89
    assert list(inspect.signature(_C.ops.attention_fp16).parameters) == ["q", "k", "v", "o", "scale"]   # ops.h:112-118
    for name in ("set_log_level", "set_cuda_stack_limit", "disable_memory_auto_release", "trim_memory", "set_faster_i2f_mode"):
        assert callable(getattr(_C.utils, name))                                           # pybind.cpp:118-123
    _C.utils.set_log_level("debug")
    _C.utils.set_cuda_stack_limit(8192)
    _C.utils.disable_memory_auto_release()
    _C.utils.set_faster_i2f_mode("enabled")
    _C.utils.trim_memory()


@pytest.fixture()
def reference_modules(monkeypatch):
    """The reference's own op / module files, imported against the shim (nothing of the reference is copied)."""
    if not (REF / "nunchaku" / "ops" / "gemm.py").exists():
        pytest.skip("reference tree not available")
    from nunchaku_b200 import _C

    saved = {k: v for k, v in sys.modules.items() if k == "nunchaku" or k.startswith("nunchaku.")}
    for k in saved:
        del sys.modules[k]
    for name in ("nunchaku", "nunchaku.ops", "nunchaku.models"):
        mod = types.ModuleType(name)
        mod.__path__ = [str(REF / name.replace(".", "/"))]
        sys.modules[name] = mod
    sys.modules["nunchaku._C"] = _C
    sys.modules["nunchaku"]._C = _C

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, REF / rel)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    mods = types.SimpleNamespace()
    load("nunchaku.utils", "nunchaku/utils.py")
    mods.quantize = load("nunchaku.ops.quantize", "nunchaku/ops/quantize.py")
    mods.gemm = load("nunchaku.ops.gemm", "nunchaku/ops/gemm.py")
    load("nunchaku.ops.gemv", "nunchaku/ops/gemv.py")
    mods.linear = load("nunchaku.models.linear", "nunchaku/models/linear.py")
    mods.fused = load("nunchaku.ops.fused", "nunchaku/ops/fused.py")
    yield mods
    for k in [k for k in sys.modules if k == "nunchaku" or k.startswith("nunchaku.")]:
        del sys.modules[k]
    sys.modules.update(saved)


def test_reference_wrappers_bind_to_the_shim(reference_modules, monkeypatch):
    from nunchaku_b200 import _C

    calls = []

    def rec_gemm(*a):
        assert len(a) == 29
        calls.append(("gemm", dict(zip(GEMM_ARGS, a))))

    def rec_quant(*a):
        assert len(a) == 8
        calls.append(("quant", dict(zip(QUANT_ARGS, a))))

    monkeypatch.setattr(_C.ops, "gemm_w4a4", rec_gemm)
    monkeypatch.setattr(_C.ops, "quantize_w4a4_act_fuse_lora", rec_quant)
    Lin = reference_modules.linear.SVDQW4A4Linear
    fc1 = Lin(128, 256, rank=32, precision="nvfp4", torch_dtype=torch.bfloat16)
    fc2 = Lin(256, 128, rank=16, precision="nvfp4", torch_dtype=torch.bfloat16)
    x = torch.zeros(2, 100, 128, dtype=torch.bfloat16)
    y = fc1(x)
    assert y.shape == (2, 100, 256)
    (k0, q), (k1, g) = calls
    assert (k0, k1) == ("quant", "gemm")
    # nunchaku/ops/quantize.py:40-51: rows padded to 256, NVFP4 scales are fp8 [K/16, M_pad], fp32 low-rank activations
    assert q["output"].shape == (256, 64) and q["output"].dtype == torch.uint8
    assert q["oscales"].shape == (8, 256) and q["oscales"].dtype == torch.float8_e4m3fn
    assert q["lora_act_out"].shape == (256, 32) and q["lora_act_out"].dtype == torch.float32
    assert q["fp4"] is True and q["fuse_glu"] is False and q["smooth"] is fc1.smooth_factor and q["lora_down"] is fc1.proj_down
    assert g["act"] is q["output"] and g["ascales"] is q["oscales"] and g["lora_act_in"] is q["lora_act_out"]
    assert g["out"].shape == (200, 256) and g["wgt"] is fc1.qweight and g["lora_up"] is fc1.proj_up and g["bias"] is fc1.bias
    assert g["lora_scales"] == [1.0, 1.0] and g["fp4"] is True and g["alpha"] is fc1.wtscale and g["wcscales"] is fc1.wcscales
    assert g["qout"] is None and g["rotary_emb"] is None and g["out_vk"] is None and g["attn_tokens"] == 0

    calls.clear()
    reference_modules.fused.fused_gelu_mlp(x, fc1, fc2)
    kinds = [c[0] for c in calls]
    assert kinds == ["quant", "gemm", "gemm"]
    g1 = calls[1][1]
    # nunchaku/ops/fused.py:10-47: fc1's GEMM writes fc2's 4-bit input and its rank-16 activations, no bf16 `out`
    assert g1["out"] is None and g1["qout"].shape == (256, 128) and g1["oscales"].shape == (16, 256)
    assert g1["lora_down"] is fc2.proj_down and g1["lora_act_out"].shape == (256, 16) and g1["smooth_factor"] is fc2.smooth_factor
    g2 = calls[2][1]
    assert g2["act"] is g1["qout"] and g2["ascales"] is g1["oscales"] and g2["lora_act_in"] is g1["lora_act_out"]


def _layer(dev):
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import helpers as H
    from oracle import svdq_ref as R

    M, K, N = 300, 256, 384
    x = R.make_activations(M, K, seed=3)
    lin = R.make_linear(K, N, 32, fp4=True, x_absmax=x.float().abs().amax(0), seed=4, mode="svd")
    return H.to_module(lin, dev), x.to(dev), (M, K, N)


@pytest.mark.gpu
def test_shim_runs_the_reference_call_pattern():
    """What nunchaku/models/linear.py:89-132 does, spelled with the shim's positional entry points."""
    from nunchaku_b200 import _C, _lib

    dev = torch.device("cuda", 0)
    m, x, (M, K, N) = _layer(dev)
    want = m(x.view(1, M, K)).view(M, N)
    M_pad = 512
    codes = torch.empty(M_pad, K // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(K // 16, M_pad, dtype=torch.float8_e4m3fn, device=dev)
    lora = torch.empty(M_pad, 32, dtype=torch.float32, device=dev)
    _C.ops.quantize_w4a4_act_fuse_lora(x, codes, scales, m.proj_down, lora, m.smooth_factor, False, True)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    _C.ops.gemm_w4a4(codes, m.qweight, out, None, scales, m.wscales, None, None, lora, m.proj_up, None, None, None, None, None,
                     m.bias, None, None, None, False, [1.0, 1.0], False, True, m.wtscale, m.wcscales, None, None, None, 0)
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    assert torch.equal(out, want)


@pytest.mark.gpu
def test_prepared_weights_follow_the_parameters():
    """The re-tiled weights hang off ``qweight``: an in-place update re-tiles, a ``.data`` write needs the explicit
    invalidation, and deleting the layer frees them."""
    import gc

    from nunchaku_b200.ops import gemm as G

    dev = torch.device("cuda", 0)
    m, x, (M, K, N) = _layer(dev)
    y0 = m(x.view(1, M, K)).clone()
    first = m.qweight.__dict__[G._ATTR][0]
    assert m(x.view(1, M, K)) is not None and m.qweight.__dict__[G._ATTR][0] is first   # served from the cache
    b0 = m.bias.detach().clone()
    with torch.no_grad():
        m.bias.add_(1.0)                                  # bumps the version counter
    y1 = m(x.view(1, M, K))
    assert m.qweight.__dict__[G._ATTR][0] is not first
    assert torch.allclose((y1 - y0).float().mean(), torch.tensor(1.0, device=dev), atol=2e-2)
    m.bias.data.copy_(b0)                                  # bypasses the counter: stale until told
    assert torch.equal(m(x.view(1, M, K)), y1)
    m.invalidate_prepared_weights()
    assert torch.equal(m(x.view(1, M, K)), y0)
    sd = {k: v.clone() for k, v in m.state_dict().items()}
    sd["bias"] += 2.0
    m.load_state_dict(sd)
    assert G._ATTR not in m.qweight.__dict__
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    del m, first, sd
    gc.collect()
    assert torch.cuda.memory_allocated(dev) < before


def test_prepared_cache_keys_on_identity_and_version(monkeypatch):
    """Host logic of the per-parameter cache, with the device call stubbed out (no GPU)."""
    import gc
    import weakref

    from nunchaku_b200.ops import gemm as G

    made = []

    class Stub:
        key = None

    def fake_prepare(*a):
        made.append(a)
        return Stub()

    monkeypatch.setattr(G, "prepare_weights", fake_prepare)
    w = torch.zeros(8, 4, dtype=torch.int8)
    s = torch.zeros(2, 8)
    b = torch.zeros(8)
    alpha = torch.tensor([2.0])
    p0 = G.cached_prepared_weights(w, s, None, b, None, alpha, None, True)
    assert G.cached_prepared_weights(w, s, None, b, None, alpha, None, True) is p0 and len(made) == 1
    assert made[0][5] == 2.0                                   # alpha read once, as a float
    b.add_(1.0)                                                # in-place update: version changes
    p1 = G.cached_prepared_weights(w, s, None, b, None, alpha, None, True)
    assert p1 is not p0 and len(made) == 2
    b2 = b.clone()                                             # same values, another tensor object
    assert G.cached_prepared_weights(w, s, None, b2, None, alpha, None, True) is not p1
    alpha.fill_(3.0)
    G.cached_prepared_weights(w, s, None, b2, None, alpha, None, True)
    assert made[-1][5] == 3.0
    n = len(made)
    b2.data.mul_(2.0)                                          # bypasses the version counter: stale until invalidated
    G.cached_prepared_weights(w, s, None, b2, None, alpha, None, True)
    assert len(made) == n
    G.invalidate_prepared(w)
    G.cached_prepared_weights(w, s, None, b2, None, alpha, None, True)
    assert len(made) == n + 1
    ref = weakref.ref(w.__dict__[G._ATTR][0])
    made.clear()                                               # the recorder holds the tensors too
    del w
    gc.collect()
    assert ref() is None                                       # the prepared copy dies with its qweight
