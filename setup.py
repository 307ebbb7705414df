"""Packaging entry point: builds the sm_100a extension in-tree, then installs the package.

``pip install --no-build-isolation .`` compiles ``lplb_b200/csrc`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` through ``lplb_b200/_native.py`` (no GPU is
needed to build) and ships the resulting shared object as package data.  Counterpart of the
reference's ``setup.py`` (reference ``setup.py:1-50``); there is no MathDx download step.
"""

import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_lplb_native_build", Path(__file__).parent / "lplb_b200" / "_native.py")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        module.build()
        super().run()


setup(cmdclass={"build_py": BuildNative})
