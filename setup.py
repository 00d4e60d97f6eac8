"""Packaging: ``pip install -e . --no-build-isolation`` (or ``python setup.py build_ext --inplace``).

The import name is ``minisgl``; its sources live in ``deepseek-v4-sm80_b200/``.  ``build_ext`` compiles the CUDA
library for sm_100a and the host C++ library in-tree (``ops/libdsv4_b200.so``, ``ops/libdsv4_host.so``) with the same
commands as ``python deepseek-v4-sm80_b200/ops/build.py``; the ``csrc`` tree ships as package data so that an
installed copy can rebuild itself.  Mirrors the reference's setuptools packaging of its ``csrc/**`` (pyproject.toml).
"""
import os
import runpy

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
SRC = "deepseek-v4-sm80_b200"


class build_ext(Command):
    description = "compile the sm_100a CUDA library and the host library in-tree"
    user_options = [("inplace", "i", "ignored: the libraries are always built in-tree")]

    def initialize_options(self):
        self.inplace = 1

    def finalize_options(self):
        pass

    def run(self):
        mod = runpy.run_path(os.path.join(ROOT, SRC, "ops", "build.py"))
        mod["build_all"]()


class build_py_with_native(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


subpackages = ["minisgl"] + ["minisgl." + p for p in find_packages(os.path.join(ROOT, SRC))]
setup(
    name="minisgl-b200",
    version="0.1.0",
    description="B200-native (sm_100a) DeepSeek-V4-Flash serving engine",
    packages=subpackages,
    package_dir={"minisgl": SRC},
    package_data={"minisgl": ["ops/csrc/*", "ops/csrc/host/*", "ops/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    extras_require={"serve": ["fastapi", "uvicorn", "pyzmq", "msgpack", "transformers"]},
    cmdclass={"build_ext": build_ext, "build_py": build_py_with_native},
    entry_points={"console_scripts": ["minisgl=minisgl.__main__:main"]},
)
