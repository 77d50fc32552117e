"""Packaging of mist_b200.

    pip install -e .            # development install; builds the native libraries in-tree
    python setup.py build_native

The CUDA kernels (``mist_b200/csrc``, sm_100a only) and the C++ runtime (``mist_b200/runtime``) are
compiled by ``mist_b200.ops.build`` with nvcc / g++ into ``mist_b200/_native``; there is no
torch-extension step, the libraries are plain C ABIs loaded with ctypes.
"""
import os
import subprocess
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    subprocess.check_call([sys.executable, "-m", "mist_b200.ops.build"], cwd=HERE)


class BuildNative(Command):
    description = "compile the sm_100a kernels and the C++ runtime into mist_b200/_native"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


class Develop(develop):
    def run(self):
        _build_native()
        super().run()


setup(
    name="mist_b200",
    version="0.1.0",
    description="Blackwell-native distributed-training optimizer: symbolic analyzer, strategy tuner and "
                "overlap-centric executor with hand-written sm_100a kernels",
    packages=find_packages(include=["mist_b200", "mist_b200.*"]),
    package_data={"mist_b200": ["configs/**/*.yaml", "configs/*.yaml", "node_database/cache_*/*.json",
                                "_native/*.so", "csrc/*", "runtime/*", "tools/scripts/*.sh"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.4", "numpy", "sympy", "pyyaml"],
    cmdclass={"build_native": BuildNative, "build_py": BuildPy, "develop": Develop},
)
