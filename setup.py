"""Builds the two native libraries in-tree (``python setup.py build_ext --inplace`` or ``pip install -e .``):
``hotspa_ae_b200/_hsb_core*.so`` (C++ host core, pybind11) and ``hotspa_ae_b200/_hsb_kernels.so`` (CUDA kernels for
sm_100a, plain C ABI).  The real work is in ``hotspa_ae_b200/build.py``; nvcc cross-compiles without a GPU."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildNative(build_ext):
    def run(self):
        from hotspa_ae_b200 import build as B
        B.build_all(force=False)


setup(name="hotspa_ae_b200", version="0.1.0", packages=find_packages(include=["hotspa_ae_b200*", "hetu*"]),
      package_data={"hotspa_ae_b200": ["*.so", "csrc/**/*"]}, cmdclass={"build_ext": BuildNative},
      python_requires=">=3.10")
