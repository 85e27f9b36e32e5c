"""Builds the CUDA library in-tree: ``python -m separableflowthesis_b200.build``.

Everything is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); nvcc
cross-compiles without a GPU.  The result, ``csrc/libsepflow_b200.so``, exports the C ABI declared in
``include/sepflow_b200.h``.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(CSRC, "libsepflow_b200.so")
SOURCES = ["prepare.cu", "sweep.cu", "grad_gemm.cu", "attention.cu", "lookup.cu", "lookup4d.cu", "resample.cu", "c_abi.cu"]
HEADERS = ["kernels.h", "sm100_primitives.cuh", os.path.join("..", "..", "include", "sepflow_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc/*.cu`` into ``csrc/libsepflow_b200.so`` if missing or out of date."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


PYBIND_DIR = os.path.join(PKG_DIR, "pybind")
PYBIND_SRC = os.path.join(PYBIND_DIR, "memorysaver_module.cpp")
PYBIND_OUT = os.path.join(PYBIND_DIR, "MemorySaver.so")


def build_pybind_module(force: bool = False) -> str:
    """Compile ``pybind/memorysaver_module.cpp`` into ``pybind/MemorySaver.so``: a native Python module with the five
    names of the reference's pybind11 module (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112) over the C ABI.
    Host code only (g++ with torch's headers); it finds ``libsepflow_b200.so`` at import time."""
    deps = [PYBIND_SRC, os.path.join(PKG_DIR, "..", "include", "sepflow_b200.h")]
    if not force and os.path.exists(PYBIND_OUT) and all(os.path.getmtime(PYBIND_OUT) > os.path.getmtime(d) for d in deps):
        return PYBIND_OUT
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=MemorySaver",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-I", inc]
    cmd += [PYBIND_SRC, "-o", PYBIND_OUT, "-L", lib_dir, "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_python",
            "-L", os.path.join(cuda_home, "lib64"), "-lcudart", "-ldl", f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the MemorySaver module failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr[-4000:])
    return PYBIND_OUT


def load_pybind_module():
    """Import ``pybind/MemorySaver.so`` as the module ``MemorySaver`` (what the reference imports from
    ``libs/MemorySaver/build/lib``)."""
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    if not os.path.exists(PYBIND_OUT):
        raise RuntimeError(f"{PYBIND_OUT} is missing: build it with `python -m separableflowthesis_b200.build`")
    spec = importlib.util.spec_from_file_location("MemorySaver", PYBIND_OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_pybind_module(force="--force" in sys.argv))
