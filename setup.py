"""Builds the native libraries (CUDA kernels for sm_100a, the host C++ core, the C API) in-tree before packaging, so
that a wheel carries ``fastdeploy_b200/_native/*.so``. ``python setup.py build_ext --inplace`` only compiles;
``pip wheel .`` compiles and packages. nvcc must be on PATH (or under /usr/local/cuda); no GPU is needed to build."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithNative(build_py):
    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from fastdeploy_b200._native import build
        build.build_all(verbose=bool(os.environ.get("FDB200_VERBOSE_BUILD")))
        super().run()


setup(cmdclass={"build_py": BuildWithNative})
