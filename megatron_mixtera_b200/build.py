"""Builds ``libb200_decode.so`` (all sm_100a kernels + the C ABI) in-tree with nvcc, and
``libb200_decode_torch.so`` (the torch custom-op front, ``TORCH_LIBRARY(b200_decode, ...)``) with g++.

nvcc cross-compiles for sm_100a without a GPU, so this also runs on CPU-only build machines.  The torch front holds
no kernels: it links the C-ABI library (found next to it through ``$ORIGIN``) and the torch libraries of the
interpreter that builds it.
"""
from __future__ import annotations

import contextlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libb200_decode.so")
TORCH_LIB_PATH = os.path.join(PKG_DIR, "libb200_decode_torch.so")
TORCH_SRC = os.path.join(CSRC, "torch_binding.cpp")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    out = [os.path.join(PKG_DIR, "..", "include", "b200_decode.h")]
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh")):
            out.append(os.path.join(CSRC, f))
    return out


@contextlib.contextmanager
def _build_lock():
    import fcntl

    with open(os.path.join(PKG_DIR, ".build.lock"), "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    with _build_lock():  # several ranks of one job may get here at once: one compiles, the others find it done
        if not force and not needs_build():
            return LIB_PATH
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        if not os.path.exists(nvcc):
            raise RuntimeError("nvcc not found: cannot build libb200_decode.so")
        tmp = LIB_PATH + ".tmp%d" % os.getpid()
        cmd = [nvcc, *NVCC_FLAGS, "-o", tmp, os.path.join(CSRC, "b200_decode.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), file=sys.stderr)
        proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        os.replace(tmp, LIB_PATH)
        if verbose:
            print(proc.stderr, file=sys.stderr)
    return LIB_PATH


def torch_ops_need_build() -> bool:
    if not os.path.exists(TORCH_LIB_PATH):
        return True
    t = os.path.getmtime(TORCH_LIB_PATH)
    deps = [TORCH_SRC, os.path.join(PKG_DIR, "..", "include", "b200_decode.h")]
    return any(os.path.getmtime(s) > t for s in deps)


def build_torch_ops(force: bool = False) -> str:
    """Compile the torch custom-op front if it is missing or older than its source; returns its path."""
    build()
    if not force and not torch_ops_need_build():
        return TORCH_LIB_PATH
    with _build_lock():
        if not force and not torch_ops_need_build():
            return TORCH_LIB_PATH
        return _compile_torch_ops()


def _compile_torch_ops() -> str:
    import torch
    from torch.utils import cpp_extension

    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found: cannot build libb200_decode_torch.so")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in cpp_extension.include_paths() + [os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", inc]
    tmp = TORCH_LIB_PATH + ".tmp%d" % os.getpid()
    cmd += [TORCH_SRC, "-o", tmp, "-L" + PKG_DIR, "-lb200_decode", "-L" + torch_lib, "-ltorch", "-ltorch_cpu",
            "-ltorch_cuda", "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("g++ failed on torch_binding.cpp:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, TORCH_LIB_PATH)
    return TORCH_LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_torch_ops(force="--force" in sys.argv))
