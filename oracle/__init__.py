"""CPU oracle for the SVDQuant W4A4 linear hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory: it is the checker used by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline leg of ``bench.py``.  It restates, with torch/numpy on
the CPU, the arithmetic of the reference kernels

  * ``src/kernels/zgemm/gemm_w4a4.cuh``  (quantise: 85-187, 429-523, 930-1043;
    GEMM: 273-356, 832-928; quantise kernel driver: 1097-1184)
  * ``src/kernels/zgemm/gemm_base.cuh``  (activation load / GLU: 589-646, bias
    epilogue: 710-781, scale packing: 97-154, 452-468)
  * ``src/kernels/zgemm/lora.cuh``       (LoRA down: 243-353, up: 110-241)
  * ``src/kernels/zgemm/gemm_utils.cuh`` (cvt / rcp / div primitives: 206-344)
  * ``nunchaku/lora/flux/packer.py``     (weight / scale / low-rank packing)

Parity status: the reference ships no unit test, golden vector or CPU
implementation for these kernels, and its CUDA extension cannot be built in a
container without its (un-vendored) submodules, so the *arithmetic* oracle is
"parity unpinned" by reference-owned vectors.  The *layout* half is pinned:
``tests/golden/`` holds outputs of the reference's own ``NunchakuWeightPacker``
(imported from the reference tree by ``tests/golden/make_golden.py``) and
``tests/test_oracle_layouts.py`` checks ``oracle.layouts`` against them.
"""
