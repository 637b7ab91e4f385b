"""Build the C-ABI CUDA library in-tree with nvcc (sm_100a only), and the torch binding on top of it with g++."""
from __future__ import annotations

import os
import shutil
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libuniql_b200.so")
EXT_NAME = "_torch_ext"
EXT_PATH = os.path.join(PKG_DIR, EXT_NAME + ".so")
EXT_SRC = os.path.join(CSRC, "torch_binding.cpp")
HEADER = os.path.join(os.path.dirname(PKG_DIR), "include", "uniql_b200.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG_DIR), "include", "uniql_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu into libuniql_b200.so next to this file; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libuniql_b200.so")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH + ".tmp", *sources(), "-lcudart"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print(res.stderr)
    return LIB_PATH


def _ext_stale() -> bool:
    if not os.path.exists(EXT_PATH):
        return True
    t = os.path.getmtime(EXT_PATH)
    return any(os.path.getmtime(d) > t for d in (EXT_SRC, HEADER) if os.path.exists(d))


def build_torch_ext(force: bool = False) -> str:
    """Compile csrc/torch_binding.cpp into _torch_ext.so next to this file: a pybind module over ATen that calls the
    C ABI of libuniql_b200.so (found through an $ORIGIN rpath).  Host code only: g++, no nvcc."""
    build()
    if not force and not _ext_stale():
        return EXT_PATH
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found: cannot build the torch binding")
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    inc = [os.path.dirname(HEADER), *ce.include_paths(), os.path.join(cuda_home, "include"),
           sysconfig.get_paths()["include"]]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in inc], EXT_SRC, "-o", EXT_PATH + ".tmp",
           f"-L{PKG_DIR}", "-luniql_b200", "-Wl,-rpath,$ORIGIN",
           f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
           "-lc10", "-lc10_cuda", f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed on the torch binding:\n" + res.stdout + res.stderr)
    os.replace(EXT_PATH + ".tmp", EXT_PATH)
    return EXT_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_torch_ext(force="--force" in sys.argv))
