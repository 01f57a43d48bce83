"""``pip install .`` / ``python setup.py build_ext --inplace``: compiles the two native extensions in-tree
(``tensornet_b200/_ext``) with the same code path as ``python __graft_entry__.py``.  nvcc cross-compiles for
sm_100a, so no GPU is needed to build."""
import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _compile_native():
    from tensornet_b200 import _build

    _build.build_all(verbose=bool(os.environ.get("TN_BUILD_VERBOSE")))


class BuildNative(build_ext):
    def run(self):
        _compile_native()


class BuildPyWithNative(build_py):
    def run(self):
        if not os.environ.get("TN_SKIP_NATIVE_BUILD"):
            _compile_native()
        super().run()


setup(cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative})
