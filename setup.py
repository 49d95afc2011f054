"""Builds the PyTorch extension `mla_bwd_cuda` (the reference's module name, `mla_bwd/setup.py:61-78`).

    python setup.py build_ext --inplace

One binding file (checks, allocation, stream) plus the C-ABI library source with all kernels, compiled for
sm_100a only.  nvcc cross-compiles, so the build needs no GPU.
"""
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("test_operator_b200", "csrc")

setup(
    name="mla_bwd_cuda",
    version="0.2.0",
    ext_modules=[
        CUDAExtension(
            name="mla_bwd_cuda",
            sources=[os.path.join(CSRC, "mla_bwd_ext.cpp"), os.path.join(CSRC, "smla_api.cu")],
            include_dirs=[os.path.join(ROOT, "include")],
            depends=[os.path.join(CSRC, h) for h in ("sm100_ptx.cuh", "smla_kernels.cuh", "smla_index_inverse.cuh")]
            + [os.path.join("include", "smla_bwd.h")],
            extra_compile_args={
                "cxx": ["-O3", "-std=c++17"],
                "nvcc": ["-O3", "-std=c++17", "-lineinfo", "-gencode=arch=compute_100a,code=sm_100a"],
            },
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=False)},
)
