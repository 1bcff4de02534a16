"""Builds the native extension in place (`python setup.py build_ext --inplace` or `pip install -e .`).

The compile itself is `mccl_b200/_build.py` (ninja through torch.utils.cpp_extension,
`-gencode arch=compute_100a,code=sm_100a`); nvcc cross-compiles, so no GPU is needed.
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _compile():
    from mccl_b200 import _build
    _build.build(verbose=True)


class build_ext(_build_ext):
    def run(self):
        _compile()


class build_py(_build_py):
    def run(self):
        _compile()
        super().run()


setup(cmdclass={"build_ext": build_ext, "build_py": build_py}, package_data={"mccl_b200": ["_C.so", "bin/*", "*.json"]})
