"""In-tree build of the CUDA library and of the torch operator plugin.

``python -m cannbench_operator_solutions_b200.build`` compiles
``libw8a8ffn.so`` (the C-ABI library, plain CUDA runtime, no torch) for
sm_100a next to this file, then the torch plugin that registers the
``cann_bench::*`` operator schemas on top of it.  nvcc cross-compiles without
a GPU.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libw8a8ffn.so")
PLUGIN_PATH = os.path.join(PKG_DIR, "libcann_bench_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    # results depend on which multiply/add pairs round separately
    "-fmad=false",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def library_sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = library_sources()
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(PKG_DIR, "..", "include", "w8a8ffn.h")]
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest(deps):
        return LIB_PATH
    objs = []
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and os.path.exists(o) and os.path.getmtime(o) >= _newest(deps):
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", s, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for s, p in procs:
        out, _ = p.communicate()
        log.append(f"== {os.path.basename(s)}\n{out}")
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {s}")
    with open(os.path.join(obj_dir, "ptxas.log"), "a" if not force else "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-lcudart"]
    subprocess.run(cmd, check=True)
    return LIB_PATH


def build_plugin(force: bool = False) -> str:
    """Compile the torch plugin (host C++ only) against libw8a8ffn.so."""
    src = os.path.join(CSRC, "plugin", "cann_bench_ops.cpp")
    deps = [src, os.path.join(PKG_DIR, "..", "include", "w8a8ffn.h")]
    if not force and os.path.exists(PLUGIN_PATH) and os.path.getmtime(PLUGIN_PATH) >= _newest(deps):
        return PLUGIN_PATH
    import torch
    from torch.utils import cpp_extension

    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    import sysconfig

    inc += ["-isystem", sysconfig.get_paths()["include"], "-I/usr/local/cuda/include"]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        "/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
        "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", PLUGIN_PATH,
        f"-L{PKG_DIR}", "-l:libw8a8ffn.so", f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
        "-ltorch", "-L/usr/local/cuda/lib64", "-lcudart",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}",
    ]
    subprocess.run(cmd, check=True)
    return PLUGIN_PATH


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_plugin(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_PATH)
    print(PLUGIN_PATH)
