"""`python setup.py install` / `pip install .` builds the extension module `mha_manual`, as the
reference's setup.py does (shmsong/NvFuserExamples setup.py:7-18), plus the CUDA kernel library
it calls.  The kernels are compiled for sm_100a only.  For in-tree development use
`python -m nvfuserexamples_b200.build` instead (same compiler flags, no install step)."""
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

this_dir = os.path.dirname(os.path.abspath(__file__))
csrc = os.path.join("nvfuserexamples_b200", "csrc")

setup(
    name="mha_manual",
    version="0.1.0",
    packages=find_packages(include=["nvfuserexamples_b200*"]),
    ext_modules=[
        CUDAExtension(
            name="mha_manual",
            sources=[os.path.join(csrc, f) for f in
                     ("mha_manual_ext.cpp", "fmha_capi.cu", "fmha_fwd_sm100.cu", "fmha_fwd_dense_sm100.cu", "fmha_fwd_fast_sm100.cu", "fmha_bwd_sm100.cu")],
            include_dirs=[os.path.join(this_dir, "include")],
            extra_compile_args={
                "cxx": ["-O2", "-std=c++17"],
                "nvcc": ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a"],
            },
        )
    ],
    cmdclass={"build_ext": BuildExtension},
)
