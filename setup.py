"""setuptools front end: ``python setup.py build_ext --inplace`` compiles the native extension for
sm_100a next to the Python sources, ``python setup.py clean`` removes it again.

Counterpart of the reference's setup.py + cmake.py (setup.py:15-78, cmake.py:52-115); the build
itself is driven by torch_dist_ext_b200/_build.py (ninja, nvcc -gencode arch=compute_100a,code=sm_100a).
"""
import importlib.util
import os

from setuptools import Command, Extension, find_packages, setup
from setuptools.command.build_ext import build_ext

HERE = os.path.dirname(os.path.abspath(__file__))


def _builder():
    spec = importlib.util.spec_from_file_location("_tdx_build", os.path.join(HERE, "torch_dist_ext_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildExt(build_ext):
    def run(self):
        print("built", _builder().build(verbose=bool(self.verbose > 1)))


class Clean(Command):
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _builder().clean()


setup(
    name="torch_dist_ext_b200",
    version="0.1.0",
    description="Blackwell-native fused all-reduce + RMSNorm (+fp8) ops, tcgen05 GEMMs fused with their collectives",
    packages=find_packages(include=["torch_dist_ext_b200*", "torch_dist_ext"]),
    package_data={"torch_dist_ext_b200": ["_C.so", "csrc/*", "csrc/include/tdx/*"]},
    ext_modules=[Extension("torch_dist_ext_b200._C", sources=[])],
    cmdclass={"build_ext": BuildExt, "clean": Clean},
)
