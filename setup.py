"""Packaging of the B200 configurable hierarchical collectives.

The native library is built in the source tree by the package's own build
module (nvcc for sm_100a, g++ for the host half), so

    python setup.py build_ext --inplace      # same as `make build`
    pip install --no-build-isolation .       # builds, then installs the package with libchb.so and bin/chb_bench

both end up with ``libchb.so`` next to the Python sources.
"""
import importlib.util
from pathlib import Path

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
PKG = "configurable_hierarchical_allreduce_algorithms_b200"


def _native_build():
    # load the build module by path: importing the package would try to load the library it is about to build
    spec = importlib.util.spec_from_file_location("_chb_build", ROOT / PKG / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=False)


class BuildExt(Command):
    """Builds libchb.so (and the native tools) in place; there is no CPython extension module."""
    description = "build libchb.so for sm_100a in the source tree"
    user_options = [("inplace", "i", "accepted for compatibility: the build is always in place")]
    boolean_options = ["inplace"]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        print(_native_build())


class BuildPy(build_py):
    def run(self):
        _native_build()
        super().run()


setup(
    name="configurable-hierarchical-allreduce-algorithms-b200",
    version="0.1.0",
    description="Configurable hierarchical allreduce / reduce-scatter / allgather for B200 (sm_100a) over NVLink / NVSwitch",
    packages=find_packages(include=[PKG, PKG + ".*"]),
    package_data={PKG: ["libchb.so", "bin/*", "utils/*.json", "csrc/api/*.h", "csrc/boot/*.h"]},
    python_requires=">=3.10",
    install_requires=[],          # torch and numpy are expected in the environment (no index access is assumed)
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
    zip_safe=False,
)
