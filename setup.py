"""Build hook: compile the native sm_100a library before the Python files are collected.

``pip install .`` / ``pip install -e . --no-build-isolation`` run ``build_py``, which first calls
``yafsdp_b200._native.build()`` (``nvcc -gencode arch=compute_100a,code=sm_100a`` over ``csrc/*.cu`` into
``yafsdp_b200/lib/libyafsdp_b200.so``) so that the shared object ships as package data.  Everything else is declared in
``pyproject.toml``.
"""

import importlib.util
import pathlib
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = pathlib.Path(__file__).resolve().parent


def _build_native() -> None:
    # load _native.py by path: importing the package would import torch, which a build environment may lack
    spec = importlib.util.spec_from_file_location("_yafsdp_native_build", ROOT / "yafsdp_b200" / "_native.py")
    assert spec is not None and spec.loader is not None
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    try:
        path = mod.build()
        print(f"[yafsdp_b200] native library built: {path}")
    except RuntimeError as e:  # no nvcc here: the library is built on first use instead
        print(f"[yafsdp_b200] WARNING: native library not built ({e})", file=sys.stderr)


class BuildPyWithNative(build_py):
    def run(self) -> None:
        _build_native()
        super().run()


setup(cmdclass={"build_py": BuildPyWithNative})
