"""Packaging for moonep_b200.

The native library is one plain-C-ABI shared object built by nvcc for sm_100a
(``moonep_b200/_build.py``), loaded with ctypes; there is no CPython extension module.  The
``build_ext`` step below compiles it in-tree (``moonep_b200/_lib/libmoonep_b200.so``) and ships it
as package data, so ``pip install --no-build-isolation .`` and ``python setup.py build_ext
--inplace`` both leave an importable package.  (The reference's setup.py builds a pybind11
extension with torch's CUDAExtension and pins its kernel DSL, setup.py:1-77; neither applies here.)
"""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _native_build(force=False):
    # load _build.py by path: importing the package would try to load the library being built
    spec = importlib.util.spec_from_file_location("_mep_build", os.path.join(HERE, "moonep_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force, verbose=True)


class BuildNative(Command):
    description = "compile csrc/ into moonep_b200/_lib/libmoonep_b200.so with nvcc (sm_100a)"
    user_options = [("force", "f", "rebuild every object"), ("inplace", "i", "accepted for compatibility")]
    boolean_options = ["force", "inplace"]

    def initialize_options(self):
        self.force = False
        self.inplace = False

    def finalize_options(self):
        pass

    def run(self):
        _native_build(force=bool(self.force))


class BuildPyWithNative(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


setup(
    name="moonep_b200",
    version="0.1.0",
    description="B200-native expert-parallel communication framework (dispatch / combine / prefetch / "
                "grad reduce over NVLink peer memory, tcgen05 grouped GEMMs, MoE layer)",
    packages=find_packages(include=["moonep_b200", "moonep_b200.*"]),
    package_data={"moonep_b200": ["_lib/*.so", "csrc/*/*"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
    zip_safe=False,
)
