"""Build libsvdq_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch headers).

    python -m nunchaku_b200.csrc.build [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SOURCES = ["api.cu", "quantize.cu", "quantize_f16.cu", "quantize_wgt.cu", "prepare.cu", "gemm_w4a4.cu", "gemm_w4a4_f16.cu", "norm_rope.cu", "norm_rope_f16.cu", "litela.cu", "litela_f16.cu", "attention.cu",
           "peak_probe.cu"]
# the fp16 builds are the bf16 sources compiled again with the 16-bit type switched
INCLUDES = {"quantize_f16.cu": "quantize.cu", "gemm_w4a4_f16.cu": "gemm_w4a4.cu", "norm_rope_f16.cu": "norm_rope.cu", "litela_f16.cu": "litela.cu"}
LIB = os.path.join(PKG, "libsvdq_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "svdq_b200.h"))
    objs = []
    jobs = []
    for src in SOURCES:
        s = os.path.join(HERE, src)
        o = os.path.join(HERE, src.replace(".cu", ".o"))
        objs.append(o)
        deps = [s] + headers + ([os.path.join(HERE, INCLUDES[src])] if src in INCLUDES else [])
        if force or _stale(o, deps):
            cmd = [NVCC, *FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=8) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    if force or jobs or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-cudart", "static", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
