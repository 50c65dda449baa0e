"""Packaging for tensorpipe_b200 (counterpart of the reference's setup.py, which drives CMake).

The native module is built by the Makefile (host g++, nvcc for sm_100a); this file only makes
`pip install .` / `pip install -e .` run that build first and ship its result together with the
Python sources. Nothing here is needed to use the tree in place: `make -j` is enough.
"""
import os
import subprocess

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNativeFirst(build_py):
    def run(self):
        subprocess.check_call(["make", "-j", str(os.cpu_count() or 4)], cwd=HERE)
        super().run()


setup(
    name="tensorpipe_b200",
    version="0.1.0",
    description="A Blackwell-native tensor pipe: point-to-point messages of CPU and CUDA tensors",
    packages=["tensorpipe_b200"],
    py_modules=["pytensorpipe"],
    package_data={"tensorpipe_b200": ["_C*.so"]},
    python_requires=">=3.9",
    cmdclass={"build_py": BuildNativeFirst},
    zip_safe=False,
)
