"""In-tree build of the two shared objects of this package.

  libalpha_moe_b200.so   CUDA kernels + C ABI (nvcc, sm_100a only, no torch dependency)
  libalpha_moe_torch.so  torch operator registration (g++, links libtorch + the C ABI library)

Both land next to this file so that they travel with the source tree.  Counterpart of the
reference's setup.py:8-31, which builds one CUDAExtension for sm_90a.
Run as `python -m alpha_moe_b200.build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
CAPI_LIB = os.path.join(HERE, "libalpha_moe_b200.so")
TORCH_LIB = os.path.join(HERE, "libalpha_moe_torch.so")

# -arch=sm_100a would also emit a generic compute_100 PTX pass that rejects tcgen05; name the
# architecture-specific target explicitly.
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CUDA_SOURCES = ["fused_moe_launch.cu", "aux_kernels.cu"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(cmd) + "\n" + res.stdout)


def _cuda_home() -> str:
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    if not os.path.exists(os.path.join(home, "bin", "nvcc")):
        nvcc = shutil.which("nvcc")
        if nvcc is None:
            raise RuntimeError("nvcc not found; set CUDA_HOME")
        home = os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))
    return home


def build_capi(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    deps.append(os.path.join(HERE, "..", "include", "alpha_moe_b200.h"))
    if not force and _newer(CAPI_LIB, deps):
        return CAPI_LIB
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-o", CAPI_LIB, *srcs]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    _run(cmd)
    return CAPI_LIB


def build_torch_op(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "torch_interface.cpp")
    deps = [src, os.path.join(HERE, "..", "include", "alpha_moe_b200.h")]
    if not force and _newer(TORCH_LIB, deps) and _newer(TORCH_LIB, [CAPI_LIB]):
        return TORCH_LIB
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = []
    for p in cpp_extension.include_paths() + [os.path.join(_cuda_home(), "include")]:
        inc += ["-isystem", p]
    abi = int(torch.compiled_with_cxx11_abi())
    cmd = ["g++", "-O2", "-fPIC", "-shared", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           *inc, src, "-o", TORCH_LIB,
           f"-L{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu", "-lc10_cuda", "-ltorch_cuda",
           f"-L{HERE}", "-lalpha_moe_b200",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd)
    return TORCH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_capi(force=force, verbose=verbose)
    build_torch_op(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(CAPI_LIB)
    print(TORCH_LIB)
