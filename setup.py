"""Packaging: `pip install -e .` (or `python setup.py build_ext --inplace`) compiles the CUDA sources for sm_100a with
nvcc into `popxl_addons_b200/lib/libxlb200.so`, in the source tree, and installs the Python package around it."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    sys.path.insert(0, HERE)
    try:
        from popxl_addons_b200.build import build
    finally:
        sys.path.pop(0)
    print("native library:", build())


class build_ext(_build_ext):
    def run(self):
        _build_native()


class build_py(_build_py):
    def run(self):
        _build_native()
        super().run()


class build_native(Command):
    description = "compile the CUDA kernels (nvcc -gencode arch=compute_100a,code=sm_100a)"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


setup(
    name="popxl_addons_b200",
    version="0.1.0",
    description="popxl.addons programming model on B200: traced graph IR, transforms, fused sm_100a kernels",
    packages=find_packages(include=["popxl_addons_b200", "popxl_addons_b200.*"]),
    package_data={"popxl_addons_b200": ["csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "lib/*.so"]},
    python_requires=">=3.10",
    install_requires=["numpy", "torch"],
    extras_require={"dev": ["pytest", "scipy"]},
    cmdclass={"build_ext": build_ext, "build_py": build_py, "build_native": build_native},
)
