"""Builds the torch extension `moonpoly` in place (python setup.py build_ext --inplace).

The extension holds no CUDA code of its own: it links libmoonpoly_gemm.so (one directory up) and
needs only the host compiler."""
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)

setup(
    name="moonpoly",
    ext_modules=[
        CUDAExtension(
            name="moonpoly",
            sources=[os.path.join("moonpoly_torch.cpp")],
            include_dirs=[os.path.join(PKG, "..", "include")],
            library_dirs=[PKG],
            libraries=["moonpoly_gemm"],
            extra_compile_args={"cxx": ["-O2", "-std=c++17"]},
            extra_link_args=["-Wl,-rpath,$ORIGIN/.."],
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=False)},
)
