"""`pip install -e . --no-build-isolation` builds the two native libraries in-tree
(CUDA kernels for sm_100a with nvcc, the C++ planner with g++ + pybind11) before installing;
the same build is available without pip as `python -m dcp_b200.csrc.build`."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from dcp_b200.csrc.build import build_all
        build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative}, py_modules=["dcp_cpp"])
