"""`python setup.py build_ext --inplace` (or `pip install -e .`) compiles the CUDA sources for sm_100a into
parameter_golf_b200/_C*.so with nvcc, the same in-tree build `python __graft_entry__.py` runs; everything else about the
package is declared in pyproject.toml."""
import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _compile():
    from parameter_golf_b200.ops import build
    build.build()


class build_ext(_build_ext):
    def run(self):
        _compile()


class build_py(_build_py):
    def run(self):
        _compile()          # the shared object is package data: build it before the package is collected
        super().run()


setup(cmdclass={"build_ext": build_ext, "build_py": build_py})
