"""In-tree build of the native parts: ``python -m scanscam_b200.build``.

1. ``libscanscam_b200.so`` -- the CUDA kernels and the C-ABI launch layer, compiled by nvcc
   for sm_100a only (no torch involved).  With ``--checked`` also
   ``libscanscam_b200_checked.so``: the same library with device-side index tests.
2. ``scanscam_ext*.so``    -- the PyTorch extension module, a thin C++ client of (1).

Both land next to this file so that they are found by ``import scanscam_b200`` without any
installation step.  nvcc cross-compiles; no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libscanscam_b200.so")
LIB_CHECKED = os.path.join(HERE, "libscanscam_b200_checked.so")
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _cuda_sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))) + [
        os.path.join(INCLUDE, "scanscam_b200.h")]


def build_library(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """nvcc -> libscanscam_b200.so (C-ABI, sm_100a).  ``checked``: the same sources with -DSSB_CHECKED
    (device-side index tests that report through the status word instead of faulting) ->
    libscanscam_b200_checked.so; select it at run time with SCANSCAM_B200_LIB=<that path>."""
    srcs = _cuda_sources()
    lib = LIB_CHECKED if checked else LIB
    if not force and _newer(lib, srcs):
        return lib
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           *(["-DSSB_CHECKED"] if checked else []), "-o", lib, os.path.join(CSRC, "scanscam_b200.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return lib


def ext_path() -> str | None:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    for name in (f"scanscam_ext{suffix}", "scanscam_ext.so"):
        p = os.path.join(HERE, name)
        if os.path.exists(p):
            return p
    return None


def build_extension(force: bool = False, verbose: bool = False) -> str:
    """g++ -> scanscam_ext.so (pybind11 module against torch's headers), linked to the library."""
    src = os.path.join(CSRC, "torch_ext.cpp")
    deps = [src, os.path.join(INCLUDE, "scanscam_b200.h")]
    existing = ext_path()
    if not force and existing and _newer(existing, deps):
        return existing
    import torch
    from torch.utils.cpp_extension import CUDA_HOME, include_paths

    cuda_home = CUDA_HOME or "/usr/local/cuda"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    out = os.path.join(HERE, "scanscam_ext.so")
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-fPIC", "-std=c++17", "-shared", "-DTORCH_EXTENSION_NAME=scanscam_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{INCLUDE}"]
    for inc in include_paths() + [os.path.join(cuda_home, "include"), sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", out, f"-L{HERE}", "-lscanscam_b200", "-Wl,-rpath,$ORIGIN",
            f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return out


def build_all(force: bool = False, verbose: bool = False, checked: bool = False) -> None:
    build_library(force, verbose)
    build_extension(force, verbose)
    if checked:
        build_library(force, verbose, checked=True)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv)
    print(LIB)
    print(ext_path())
    if "--checked" in sys.argv:
        print(LIB_CHECKED)
