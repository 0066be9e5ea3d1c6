"""Packaging of catch_b200: builds the two native libraries in the source tree with the generated ninja file
(``catch_b200/_build.py``) and packages them with the Python sources.

    python setup.py build_ext --inplace      # same as python -m catch_b200._build
    python setup.py bdist_wheel              # wheel with the built libraries inside
    python setup.py clean                    # removes build/ and the built libraries

Environment switches (see ``catch_b200/_build.py``): ``DEBUG``, ``CATCH_B200_BUILD_ASAN``, ``CATCH_B200_BUILD_TEST``,
``MAX_JOBS``, ``NVCC``, ``CATCH_B200_CXX``.  The reference drives CMake from setup.py the same way
(setup.py:77-81,219-252 of the reference).
"""
import importlib.util
import os
import shutil
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _builder():
    spec = importlib.util.spec_from_file_location("_catch_b200_build", os.path.join(ROOT, "catch_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class NinjaBuildExt(build_ext):
    """The extension list is empty for setuptools; the native libraries come from the ninja build."""

    def run(self):
        _builder().build(verbose=bool(self.verbose and self.verbose > 1))


class BuildPyWithNative(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


class Clean(Command):
    description = "remove build/ and the built native libraries"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        b = _builder()
        for path in (b.BUILD, ):
            if os.path.isdir(path):
                shutil.rmtree(path)
        for path in (b.DEVICE_LIB, b.HOST_LIB, b.PKG / "lib" / "b200_runtime_test"):
            if os.path.exists(path):
                os.remove(path)


def _version():
    import re

    with open(os.path.join(ROOT, "catch_b200", "__init__.py")) as f:
        return re.search(r'__version__ = "([^"]+)"', f.read()).group(1)


setup(
    name="catch_b200",
    version=_version(),
    description="Out-of-tree PyTorch device backend for NVIDIA B200 (sm_100a): tcgen05 / TMA kernels, peer-memory collectives",
    packages=find_packages(include=["catch_b200", "catch_b200.*"]),
    package_data={"catch_b200": ["*.so", "lib/*.so", "lib/b200_runtime_test"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.11"],
    cmdclass={"build_ext": NinjaBuildExt, "build_py": BuildPyWithNative, "clean": Clean},
    zip_safe=False,
)
