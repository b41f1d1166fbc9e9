"""Builds libnvfp4_b200.so (sm_100a only) in-tree with nvcc.

    python nanogpt-120a_b200/build.py [--force] [--verbose]

The quantizer translation unit is compiled with -fmad=false: its arithmetic must round
exactly like the reference's device code (no multiply-add contraction).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnvfp4_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

UNITS = [
    # (source, extra flags)
    ("quant_kernels.cu", ["-fmad=false"]),
    ("gemm_tcgen05.cu", []),
    ("api.cu", []),
    ("tensor_amax_static.cu", []),
    ("checkpoint.cu", []),
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the NVFP4 library cannot be built")
    return nvcc


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "nvfp4_b200.h"))
    objs = []
    for src, extra in UNITS:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", src_path, "-o", obj]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
                print(" ".join(cmd), flush=True)
            subprocess.check_call(cmd)
    if force or _stale(LIB, objs):
        tmp = LIB + ".tmp"
        cmd = [nvcc, *ARCH, "-shared", "-o", tmp, *objs]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        os.replace(tmp, LIB)  # readers see the old library or the new one, never a partial file
    return LIB


STEP_LIB = os.path.join(HERE, "libnvfp4_b200_step.so")


def build_step_library(force: bool = False) -> str:
    """Compiles the C++ training-step driver (include/nvfp4_b200_step.hpp behind the C ABI of
    include/nvfp4_b200_step.h) into libnvfp4_b200_step.so next to the kernel library."""
    root = os.path.abspath(os.path.join(HERE, ".."))
    include = os.path.join(root, "include")
    src = os.path.join(HERE, "host", "step_capi.cpp")
    deps = [src, build()] + [os.path.join(include, f) for f in ("nvfp4_b200.h", "nvfp4_b200.hpp", "nvfp4_b200_step.h",
                                                                "nvfp4_b200_step.hpp")]
    if force or _stale(STEP_LIB, deps):
        subprocess.check_call([_nvcc(), *ARCH, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-I", include, src, "-o",
                               STEP_LIB, "-L", HERE, "-lnvfp4_b200", "-ldl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"])
    return STEP_LIB


def build_cpp_driver(force: bool = False) -> str:
    """Compiles tests/cpp/mlp_layer_driver.cpp (a C++ caller of include/nvfp4_b200.hpp that walks one MLP
    block forward and backward) against the in-tree library; returns the binary's path."""
    root = os.path.abspath(os.path.join(HERE, ".."))
    src = os.path.join(root, "tests", "cpp", "mlp_layer_driver.cpp")
    out_dir = os.path.join(root, "tests", "cpp", "build")
    exe = os.path.join(out_dir, "mlp_layer_driver")
    include = os.path.join(root, "include")
    deps = [src, os.path.join(include, "nvfp4_b200.hpp"), os.path.join(include, "nvfp4_b200.h"), build()]
    if force or _stale(exe, deps):
        os.makedirs(out_dir, exist_ok=True)
        subprocess.check_call([_nvcc(), *ARCH, "-O2", "-std=c++17", "-I", include, src, "-o", exe, "-L", HERE,
                               "-lnvfp4_b200", "-Xlinker", "-rpath", "-Xlinker", HERE])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_step_library(force="--force" in sys.argv))
    print(build_cpp_driver(force="--force" in sys.argv))
