"""Build recipe of librode_b200.so (nvcc, sm_100a) and of the torch binding.

    python -m rode_b200.build            # library + torch extension, in-tree
    python -m rode_b200.build --lib      # library only

Everything is built in-tree, next to this file, so that the binaries travel with the
source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "librode_b200.so")
SOURCES = ["rode_host.cu", "rode_preprocess.cu", "rode_hot_columns.cu", "rode_spmm.cu", "rode_sddmm.cu"]
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr",
]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into rode_b200/librode_b200.so (cross-compiles without a GPU)."""
    if not force and _newer(LIB, _deps()):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-shared", "-I", INCLUDE, "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB


def build_torch_extension(force: bool = False) -> str:
    """Compile the torch binding rode_sddmm_cuda (C++ only; links librode_b200.so)."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = os.path.join(PKG, "rode_sddmm_cuda" + suffix)
    src = os.path.join(PKG, "torch_ext", "rode_sddmm_cuda.cpp")
    if not force and _newer(target, [src, LIB] + _deps()):
        return target
    build_library()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], INCLUDE,
                                           os.path.join(cuda_home, "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cxx = os.environ.get("RODE_CXX", "/usr/bin/g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=rode_sddmm_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for i in inc:
        cmd += ["-I", i]
    cmd += [src, "-o", target, "-L", PKG, "-lrode_b200", "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10",
            "-ltorch_python", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the torch extension failed:\n" + res.stdout + res.stderr)
    return target


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if "--lib" not in sys.argv:
        build_torch_extension(force="--force" in sys.argv)
    print("built", LIB)
