"""Generate the layout golden vectors from the reference's own Python packer.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/nunchaku  tests/golden/packer_golden.npz

It imports ``nunchaku/lora/flux/packer.py`` by file path (the package itself
cannot be imported without its compiled extension), feeds seeded tensors to
``NunchakuWeightPacker`` and stores inputs and outputs.  bf16 tensors are
stored as their int16 bit patterns, fp8 as uint8.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch


def load_reference_packer(ref_root: Path):
    for name in ("nunchaku", "nunchaku.lora", "nunchaku.lora.flux"):
        mod = types.ModuleType(name)
        mod.__path__ = [str(ref_root / name.replace(".", "/"))]
        sys.modules[name] = mod

    def load(name: str, rel: str):
        spec = importlib.util.spec_from_file_location(name, ref_root / rel)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    load("nunchaku.utils", "nunchaku/utils.py")
    load("nunchaku.lora.flux.utils", "nunchaku/lora/flux/utils.py")
    return load("nunchaku.lora.flux.packer", "nunchaku/lora/flux/packer.py")


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def main(ref_root: str, out_path: str) -> None:
    packer_mod = load_reference_packer(Path(ref_root))
    packer = packer_mod.NunchakuWeightPacker(bits=4)
    g = torch.Generator().manual_seed(1234)
    N, K, R = 256, 256, 32
    out: dict[str, np.ndarray] = {}

    codes = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int32)
    out["wgt_codes_in"] = codes.numpy().astype(np.int8)
    out["wgt_codes_packed"] = packer.pack_weight(codes.clone()).view(torch.uint8).numpy()

    ws = (torch.rand(N, K // 64, generator=g) + 0.01).to(torch.bfloat16)
    out["wscales_in"] = bits16(ws)  # [N, K/64]
    out["wscales_packed"] = bits16(packer.pack_scale(ws.clone(), group_size=64))  # [K/64, N]

    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    out["vector_in"] = bits16(bias)
    out["vector_packed"] = bits16(packer.pack_scale(bias.clone().view(-1, 1), group_size=-1))

    ms = (torch.rand(N, K // 16, generator=g) * 400).to(torch.bfloat16)
    out["wmscales_in"] = ms.to(torch.float8_e4m3fn).view(torch.uint8).numpy()  # [N, K/16]
    out["wmscales_packed"] = packer.pack_scale(ms.clone(), group_size=16).view(torch.uint8).numpy()  # [K/16, N]

    up = torch.randn(N, R, generator=g).to(torch.bfloat16)
    out["lora_up_in"] = bits16(up)
    out["lora_up_packed"] = bits16(packer.pack_lowrank_weight(up.clone(), down=False))
    down = torch.randn(R, K, generator=g).to(torch.bfloat16)
    out["lora_down_in"] = bits16(down)  # logical [R, K]
    out["lora_down_packed"] = bits16(packer.pack_lowrank_weight(down.clone(), down=True))  # [K, R]

    # the documented lane maps (gemm_base.cuh:100-112): index-encoding inputs
    idx = torch.arange(128, dtype=torch.float32).to(torch.bfloat16)
    out["vector_index_packed"] = packer.pack_scale(idx.view(-1, 1), group_size=-1).to(torch.float32).numpy().astype(np.int16)

    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
