"""Packaging: the Python package plus the two in-tree native libraries.

``python setup.py build_ext --inplace`` (or any ``pip install``) compiles
``csrc/sm100/*.cu`` for sm_100a with nvcc and ``csrc/cpu/*.cpp`` with g++ into
``kernel_align_b200/_lib`` through ``kernel_align_b200/_build.py``; every sub-package is a real
package (the reference's setup.py:6 silently dropped four of its six).
"""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _native_build():
    spec = importlib.util.spec_from_file_location("_ka_build", os.path.join(HERE, "kernel_align_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all()


class BuildNative(Command):
    description = "compile the sm_100a and CPU libraries in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _native_build()


class BuildPyWithNative(build_py):
    def run(self):
        _native_build()
        super().run()


setup(
    packages=find_packages(include=["kernel_align_b200", "kernel_align_b200.*"]),
    package_data={"kernel_align_b200": ["_lib/*.so"]},
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
    zip_safe=False,
)
