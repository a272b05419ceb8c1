"""Builds the sm_100a CUDA library in-tree with nvcc and installs the Python host layer.

    python setup.py build_ext --inplace      # produces stickbreaking_attention_b200/libsb_b200.so
"""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_lib():
    spec = importlib.util.spec_from_file_location(
        "_sb_b200_build", os.path.join(HERE, "stickbreaking_attention_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


class BuildExt(Command):
    description = "compile libsb_b200.so with nvcc (sm_100a)"
    user_options = [("inplace", "i", "kept for the usual spelling; the library is always built in-tree")]

    def initialize_options(self):
        self.inplace = 1

    def finalize_options(self):
        pass

    def run(self):
        print("built", _build_lib())


class BuildPy(build_py):
    def run(self):
        _build_lib()
        super().run()


setup(
    name="stickbreaking_attention_b200",
    version="0.1.0",
    description="Stick-breaking attention for NVIDIA B200 (sm_100a), hand-written CUDA behind a C ABI",
    packages=find_packages(include=["stickbreaking_attention_b200*"]),
    package_data={"stickbreaking_attention_b200": ["libsb_b200.so", "csrc/*"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
)
