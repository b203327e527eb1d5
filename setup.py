"""Packaging of moonep_b200 (and the ``moonep_td`` import-name shim).

The native library is built in-tree with nvcc for sm_100a (``python -c "import __graft_entry__ as g; g.build()"`` or
lazily on first use, see ``moonep_b200/ops/_lib.py``); ``python setup.py build_native`` does the same from here so
that a wheel carries ``moonep_b200/lib/libmoonep_b200.so``.
"""

import os
import sys

from setuptools import Command, find_packages, setup


class BuildNative(Command):
    description = "compile moonep_b200/csrc/*.cu into moonep_b200/lib/libmoonep_b200.so (needs nvcc, no GPU)"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from moonep_b200.ops import _lib

        _lib.build(force=True)


setup(
    name="moonep-b200",
    version="0.1.0",
    description="Load-balanced expert-parallel MoE communication and expert GEMMs for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["moonep_b200", "moonep_b200.*", "moonep_td", "moonep_td.*"]),
    package_data={"moonep_b200": ["csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "lib/*.so"]},
    python_requires=">=3.11",
    install_requires=["torch>=2.6", "numpy"],
    cmdclass={"build_native": BuildNative},
)
