"""Installs the B200 build of the reference's Python surface: `pip install -e . --no-build-isolation` (the command
the reference documents, README.md:6-10 there) yields the modules `alpha_moe` (importing it registers
torch.ops.alpha_moe.fused_moe_w8a8_up_down), `alpha_moe_ops`, the package `alpha_moe_python` and the implementation
package `alpha_moe_b200` with its two shared objects.  Counterpart of the reference's setup.py:8-31, which builds one
CUDAExtension for sm_90a; here the libraries are built in-tree for sm_100a by alpha_moe_b200/build.py (nvcc with
-gencode arch=compute_100a,code=sm_100a for the C ABI library, g++ against libtorch for the operator library) as part
of the build_py / build_ext / develop steps."""
import os
import sys

import setuptools
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _build_native():
    from alpha_moe_b200 import build as native
    native.build_all(force=False)


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


class BuildExt(build_ext):
    def run(self):
        _build_native()
        super().run()


if __name__ == "__main__":
    setuptools.setup(
        name="alpha_moe_python",
        version="0.1.0",
        description="Fused W8A8 MoE layer for NVIDIA B200 (sm_100a) behind torch.ops.alpha_moe.fused_moe_w8a8_up_down",
        packages=["alpha_moe_python", "alpha_moe_b200"],
        py_modules=["alpha_moe", "alpha_moe_ops"],
        package_data={"alpha_moe_b200": ["*.so", "csrc/*"]},
        include_package_data=True,
        python_requires=">=3.10",
        cmdclass={"build_py": BuildPy, "build_ext": BuildExt},
    )
