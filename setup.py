"""Packaging hook: compiles the sm_100a kernel library with nvcc while building the package.

``pip install -e .`` / ``python setup.py build_py`` run :func:`dice_embeddings_b200.ops._lib.build`, which compiles
``csrc/*.cu`` into ``dice_embeddings_b200/ops/libdice_b200.so``.  Without nvcc the Python package is still
installed; it then runs the PyTorch paths only and reports the missing library when a kernel is requested.
The metadata lives in ``pyproject.toml``.
"""
import importlib.util
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    """Import ``ops/_lib.py`` by path: importing the package would pull in torch during the build."""
    spec = importlib.util.spec_from_file_location("_dice_b200_lib", os.path.join(ROOT, "dice_embeddings_b200", "ops",
                                                                                 "_lib.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildWithKernels(build_py):
    def run(self):
        try:
            path = _load_builder().build()
            print("kernel library:", path)
        except (RuntimeError, FileNotFoundError) as exc:
            print("warning: the kernel library was not built:", str(exc).splitlines()[0], file=sys.stderr)
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
