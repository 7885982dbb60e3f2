"""Packaging of recsdk_b200.  The native parts (``csrc/cuda`` -> ``recsdk_b200/_C_cuda.so`` with
``nvcc -gencode arch=compute_100a,code=sm_100a``; ``csrc/host`` -> the pybind11 module ``recsdk_b200/_C_host*.so``) are built
in-tree by ``recsdk_b200/_build.py``; ``build_ext`` / ``build_py`` call it, so ``pip install .`` and
``python setup.py build_ext --inplace`` both leave the binaries beside the Python sources."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py as _build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _build_native(force: bool = False) -> None:
    from recsdk_b200 import _build

    _build.build_all(force=force, verbose=True)


class build_ext(Command):
    description = "build the sm_100a kernel library and the host engines in-tree"
    user_options = [("inplace", "i", "accepted for compatibility (the build is always in-tree)"), ("force", "f", "rebuild everything")]

    def initialize_options(self):
        self.inplace, self.force = 1, 0

    def finalize_options(self):
        pass

    def run(self):
        _build_native(bool(self.force))


class build_py(_build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="recsdk_b200",
    version="0.2.0",
    description="B200-native recommendation framework: sharded and dynamic embeddings, HSTU, multi-tier embedding cache, KV-cache manager",
    packages=find_packages(include=["recsdk_b200", "recsdk_b200.*"]),
    package_data={"recsdk_b200": ["*.so"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    cmdclass={"build_ext": build_ext, "build_py": build_py},
)
