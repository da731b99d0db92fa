"""Times of the row-wise kernels either side of the W4A4 linears against their algorithmic HBM bytes.

    python -m nunchaku_b200.models.rowwise_bench [--steps 20]

Prints one JSON line: microseconds per call (CUDA events over back-to-back calls; a stand-alone launch carries 8-10 us of
launch gap) and algorithmic GB/s for RMSNorm + RoPE on a FLUX QKV output [4608, 9216], LayerNorm + modulation on
[4608, 3072] and ReLU linear attention on a SANA QKV output [4, 1024, 6912].
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _lib
from ..ops import layernorm_modulate, litela_attention, qk_norm_rope
from .mlp_bench import timed


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    g = torch.Generator(device="cuda").manual_seed(0)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    res = {}

    S, heads = 4608, 24
    qkv = torch.randn(1, S, 3 * heads * 128, generator=g, **bf)
    w = torch.ones(128, **bf)
    ang = torch.rand(S, 64, device="cuda", generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    us = timed(lambda: qk_norm_rope(qkv, w, w, cos, sin, heads), args.steps)
    byt = S * (8 * heads * 128 + 512)
    res["qk_norm_rope"] = {"us": round(us, 1), "GBps": round(byt / us / 1e3, 1), "shape": [S, 3 * heads * 128]}

    x = torch.randn(1, S, 3072, generator=g, **bf)
    sc, sh = torch.randn(1, 3072, generator=g, **bf) * 0.1, torch.randn(1, 3072, generator=g, **bf) * 0.1
    us = timed(lambda: layernorm_modulate(x, sc, sh), args.steps)
    byt = S * 3072 * 4
    res["layernorm_modulate"] = {"us": round(us, 1), "GBps": round(byt / us / 1e3, 1), "shape": [S, 3072]}

    B, T, lh = 4, 1024, 72
    q = torch.randn(B, T, 3 * lh * 32, generator=g, **bf)
    us = timed(lambda: litela_attention(q, lh), args.steps)
    byt = B * T * lh * 32 * 8
    res["litela_attention"] = {"us": round(us, 1), "GBps": round(byt / us / 1e3, 1), "shape": [B, T, 3 * lh * 32]}
    torch.cuda.synchronize()
    assert _lib.device_status() == (0, 0)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
