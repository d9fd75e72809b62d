"""Builds the native extension in-tree with ``build.py`` (ninja + nvcc for sm_100a) before the
Python package is collected, so that ``pip install .`` / ``pip install -e .`` ship
``pplx_garden/_native*.so`` and ``pplx_garden/libpplx_noalloc.so``."""

import subprocess
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNativeFirst(build_py):
    def run(self) -> None:
        root = Path(__file__).resolve().parent
        subprocess.run([sys.executable, str(root / "build.py")], check=True, cwd=root)
        super().run()


setup(cmdclass={"build_py": BuildNativeFirst})
