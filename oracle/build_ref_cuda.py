"""Builds the reference's own MemorySaver CUDA extension (libs/MemorySaver/src, the five pybind functions of
MemorySaver_cuda.cpp:105-112) from the sources where they lie in a checkout of the reference, into
``oracle/_ref/MemorySaver.so``.  Test infrastructure: on a GPU box the parity tests use it as a second oracle and
the bench can time it beside this library; nothing in the product imports it.  No reference source is copied.

    python oracle/build_ref_cuda.py /path/to/SeparableFlowThesis

The recipe is the four source files handed to nvcc (one process each) with torch's include and library paths; the
reference's setup.py is not run.  Compiled for sm_100a; takes several minutes.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "MemorySaver.so")
SOURCES = ["MemorySaver_cuda.cpp", "MemorySaver_kernel_forward.cu", "MemorySaver_kernel_max_avg_argmax_backward.cu",
           "MemorySaver_kernel_compression_backward.cu"]


def build(ref_root: str, force: bool = False) -> str:
    src_dir = os.path.join(ref_root, "libs", "MemorySaver", "src")
    srcs = [os.path.join(src_dir, f) for f in SOURCES]
    if not all(os.path.exists(f) for f in srcs):
        raise FileNotFoundError(f"reference sources not found under {src_dir}")
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) > os.path.getmtime(f) for f in srcs):
        return OUT
    from torch.utils import cpp_extension
    import torch
    os.makedirs(OUT_DIR, exist_ok=True)
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-Xcompiler", "-fPIC",
             "-DTORCH_EXTENSION_NAME=MemorySaver", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        flags += ["-I", inc]
    # one nvcc per source file, side by side (torch's headers make each of them minutes long), then one link
    objs = [os.path.join(OUT_DIR, os.path.splitext(f)[0] + ".o") for f in SOURCES]
    procs = [subprocess.Popen([nvcc, *flags, "-x", "cu", "-c", src, "-o", obj], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for src, obj in zip(srcs, objs)]
    for proc, src in zip(procs, srcs):
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out[-4000:]}")
    link = [nvcc, "-shared", *objs, "-L", lib_dir, "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda",
            "-ltorch_cuda", "-Xlinker", "-rpath", "-Xlinker", lib_dir, "-o", OUT]
    res = subprocess.run(link, capture_output=True, text=True)
    for obj in objs:
        if os.path.exists(obj):
            os.remove(obj)
    if res.returncode != 0:
        raise RuntimeError("linking the reference extension failed:\n" + res.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python oracle/build_ref_cuda.py /path/to/SeparableFlowThesis [--force]")
    print(build(sys.argv[1], force="--force" in sys.argv))
