"""`pip install .`: runs the in-tree build (nvcc for sm_100a, g++ for the PyTorch extension) and
packages `scanscam_b200` with the two libraries it produced.

The counterpart of the reference's setup.py (setup.py:1-33), which lets
`torch.utils.cpp_extension` pick architectures from the environment; here the kernels are built
for `arch=compute_100a,code=sm_100a` only, by `scanscam_b200/build.py`, and the PyTorch extension
is a thin client of the C-ABI library that sits next to it (`RUNPATH=$ORIGIN`).
"""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_ssb_build", os.path.join(HERE, "scanscam_b200", "build.py"))
        native = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(native)  # build.py imports nothing from the package
        native.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative})
