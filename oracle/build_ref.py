"""Compile the reference's own INT4 W4A4 kernels into ``oracle/_ref/libnunchaku_ref_int4.so`` (TEST INFRASTRUCTURE).

    python -m oracle.build_ref [--force]

Three translation units, compiled with nvcc for sm_100a straight from where they lie in the reference tree (nothing is
copied, the reference's own build system is not run):

  * ``src/kernels/zgemm/gemm_w4a4_launch_bf16_int4.cu``: the explicit instantiation of
    ``GEMM_W4A4_Launch<GEMMConfig_W4A4_BF16, false>`` (quantiser, GEMM with every epilogue, ``vk_mul_q``);
  * ``src/kernels/zgemm/gemm_w4a4_launch_fp16_int4.cu``: the same for ``GEMMConfig_W4A4_FP16``;
  * ``oracle/ref_int4_shim.cu``: a C-ABI wrapper around it (raw device pointers -> the reference's ``Tensor``).

The reference's ``common.h`` includes spdlog, an un-vendored submodule of the reference; a header-only copy of spdlog
ships with the ``flashinfer`` wheel of this image and is used instead (logging only, no arithmetic).  The flags are the
reference's (``setup.py:104-130``) minus its arch list.  The NVFP4 instantiations are not built: those kernels run on
sm_120a only and trap elsewhere.  The library needs a GPU to run; building does not.  Returns None when the reference
tree or the spdlog headers are missing (the GPU box has neither: it uses the prebuilt file).
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libnunchaku_ref_int4.so")
REFERENCE = os.environ.get("NUNCHAKU_REFERENCE", "/root/reference")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _spdlog_include() -> str | None:
    spec = importlib.util.find_spec("flashinfer")
    if spec is None or not spec.submodule_search_locations:
        return None
    p = os.path.join(list(spec.submodule_search_locations)[0], "data", "spdlog", "include")
    return p if os.path.isdir(os.path.join(p, "spdlog")) else None


def build(force: bool = False, verbose: bool = False) -> str | None:
    launch = os.path.join(REFERENCE, "src", "kernels", "zgemm", "gemm_w4a4_launch_bf16_int4.cu")
    shim = os.path.join(HERE, "ref_int4_shim.cu")
    if not os.path.exists(launch):
        return LIB if os.path.exists(LIB) else None
    spdlog = _spdlog_include()
    if spdlog is None:
        return LIB if os.path.exists(LIB) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    flags = [
        "-DENABLE_BF16=1", "-DBUILD_NUNCHAKU=1", "-std=c++20", "-UNDEBUG", "-O2", "-Xcudafe", "--diag_suppress=20208",
        "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
        "-U__CUDA_NO_HALF2_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__", "--expt-relaxed-constexpr",
        "--expt-extended-lambda", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
        "-I", os.path.join(REFERENCE, "src"), "-I", spdlog,
    ]
    jobs = []
    objs = []
    launch_f16 = os.path.join(REFERENCE, "src", "kernels", "zgemm", "gemm_w4a4_launch_fp16_int4.cu")
    for src, name in ((launch, "launch_bf16_int4.o"), (launch_f16, "launch_fp16_int4.o"), (shim, "shim.o")):
        obj = os.path.join(OUT_DIR, name)
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < os.path.getmtime(src):
            jobs.append([NVCC, *flags, "-c", src, "-o", obj])

    def run(cmd):
        return cmd, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=3) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"reference build failed for {cmd[-3]}")
    if jobs or not os.path.exists(LIB):
        r = subprocess.run([NVCC, "-shared", "-cudart", "static", "-o", LIB, *objs], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("reference link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
