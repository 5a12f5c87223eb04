"""Builds the native parts in-tree (nvcc for sm_100a, g++ for the host libraries and the torch
extension) before the Python package is collected, so that a wheel carries the shared objects.

    pip install --no-build-isolation .
"""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNativeFirst(build_py):
    def run(self):
        import os
        import sys

        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from rocm_systems_b200.utils import build

        build.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNativeFirst})
