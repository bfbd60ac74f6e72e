"""Packaging: ``pip install --no-build-isolation -e .`` (or ``python setup.py build_ext --inplace``) compiles the native
parts in-tree with ``fuselink_b200.build`` -- the CUDA extension for sm_100a, the ncclNet plugin, the monitor daemon and
the plugin harness -- and installs the Python package around them."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(_build_ext):
    """Runs the project's own build driver instead of setuptools' compiler logic."""

    def run(self):
        sys.path.insert(0, ROOT)
        from fuselink_b200 import build
        build.build_all()


class BuildSanitized(Command):
    description = "build the host-side code with sanitizers (address,undefined | thread)"
    user_options = [("kind=", None, "sanitizer list")]

    def initialize_options(self):
        self.kind = "address,undefined"

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, ROOT)
        from fuselink_b200 import build
        print(build.build_sanitized(self.kind))


setup(
    name="fuselink_b200",
    version="0.1.0",
    description="Blackwell-native multi-path GPU communication framework (ncclNet plugin, cuMem regions, fused sm_100a kernels)",
    packages=find_packages(include=["fuselink_b200", "fuselink_b200.*"]),
    package_data={"fuselink_b200": ["_C.so", "lib/*", "csrc/**/*"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildNative, "build_sanitized": BuildSanitized},
    entry_points={"console_scripts": ["fuselink-serving=fuselink_b200.serving.__main__:main",
                                      "fuselink-metrics=fuselink_b200.utils.metrics:main"]},
)
