"""The C-ABI library loads, exports every symbol include/svdq_b200.h declares, and the ctypes
mirror of its structs has the layout the C compiler gives them (no GPU, no compute calls)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "svdq_b200.h")


@pytest.fixture(scope="module")
def lib():
    from nunchaku_b200.csrc.build import build

    build()
    from nunchaku_b200 import _lib

    return _lib


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(svdq_[a-z0-9_]+)\s*\(", src)))


def test_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 9
    cdll = lib.load()
    for n in names:
        assert hasattr(cdll, n), f"{n} is declared in the header but not exported"
        assert n in lib.EXPORTS, f"{n} has no ctypes prototype"
    assert cdll.svdq_version() >= 100


def test_struct_layout_matches_c(lib, tmp_path):
    structs = {
        "svdq_quantize_args": lib.QuantizeArgs,
        "svdq_prepared_weights": lib.PreparedWeights,
        "svdq_weights_args": lib.WeightsArgs,
        "svdq_gemm_args": lib.GemmArgs,
        "svdq_relayout_args": lib.RelayoutArgs,
        "svdq_norm_rope_args": lib.NormRopeArgs,
        "svdq_ln_modulate_args": lib.LnModulateArgs,
        "svdq_gate_residual_args": lib.GateResidualArgs,
        "svdq_litela_args": lib.LiteLAArgs,
        "svdq_attention_args": lib.AttentionArgs,
        "svdq_quantize_wgt_args": lib.QuantizeWgtArgs,
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, cls in structs.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines.append("return 0;}")
    c = tmp_path / "layout.c"
    c.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-o", str(exe), str(c)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    got = dict(l.split() for l in out.strip().splitlines())
    for cname, cls in structs.items():
        assert int(got[cname]) == ctypes.sizeof(cls)
        for fname, _ in cls._fields_:
            assert int(got[f"{cname}.{fname}"]) == getattr(cls, fname).offset, f"{cname}.{fname}"


def test_argument_validation_needs_no_gpu(lib):
    """Shape / pointer checks run before any CUDA call and return SVDQ_ERR_INVALID_ARGUMENT."""
    cdll = lib.load()
    assert cdll.svdq_quantize_w4a4_act_fuse_lora(None, None) == lib.SVDQ_ERR_INVALID_ARGUMENT
    a = lib.QuantizeArgs(input=16, codes=16, scales=16, lora_act=16, smooth=16, lora_down=16,
                         M=10, M_pad=100, K=128, R=32, fp4=1, fuse_glu=0, layout=0)
    assert cdll.svdq_quantize_w4a4_act_fuse_lora(ctypes.byref(a), None) == lib.SVDQ_ERR_INVALID_ARGUMENT
    assert b"multiple of 256" in cdll.svdq_last_error_string()
    a.M_pad, a.K = 256, 100
    assert cdll.svdq_quantize_w4a4_act_fuse_lora(ctypes.byref(a), None) == lib.SVDQ_ERR_INVALID_ARGUMENT
    a.K, a.input = 128, 8  # misaligned pointer
    assert cdll.svdq_quantize_w4a4_act_fuse_lora(ctypes.byref(a), None) == lib.SVDQ_ERR_INVALID_ARGUMENT
    with pytest.raises(ValueError):
        lib.check(lib.SVDQ_ERR_INVALID_ARGUMENT)
    g = lib.GemmArgs()
    assert cdll.svdq_gemm_w4a4(ctypes.byref(g), None) == lib.SVDQ_ERR_INVALID_ARGUMENT
    sizes = (ctypes.c_size_t * 5)()
    assert cdll.svdq_w4a4_prepared_bytes(21504, 3072, 32, 1, sizes) == 0
    assert list(sizes) == [21504 * 3072 // 2, 21504 * 3072 // 16, 21504 * 32 * 4, 21504 * 4, 21504 * 4]
    assert cdll.svdq_w4a4_prepared_bytes(100, 3072, 32, 1, sizes) == lib.SVDQ_ERR_INVALID_ARGUMENT


def test_quantiser_launch_plan(lib):
    """Cluster size along K and pipeline depth chosen on the host (148 SMs)."""
    cdll = lib.load()
    cdll.svdq_quantize_plan.restype = ctypes.c_int
    ks, nst, smem = ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()

    def plan(M_pad, K, R):
        rc = cdll.svdq_quantize_plan(M_pad, K, R, 148, ctypes.byref(ks), ctypes.byref(nst), ctypes.byref(smem))
        assert rc == 0
        return ks.value, nst.value, smem.value

    k, n, s = plan(4608, 3072, 32)       # 72 row blocks x cluster of 2 = 144 CTAs on 148 SMs, one wave
    assert k == 2 and n >= 4 and s <= 227 * 1024
    k, n, s = plan(36864, 3072, 32)      # batch 8: 576 row blocks already fill four waves
    assert k == 1 and s <= 227 * 1024
    k, n, s = plan(256, 128, 32)         # tiny problem: K is a single 128-column chunk
    assert k == 1 and n >= 1
    k, n, s = plan(4608, 12288, 128)
    assert s <= 227 * 1024 and n * 16384 >= 64 * 128 * 4
