"""Builds the sm_100a shared libraries of this package in-tree (binarybrain_b200/lib/).

    python -m binarybrain_b200.build            # C-ABI kernel library (+ the pybind11 host module)
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libbbcu_b200.so")

CU_SOURCES = ["runtime.cu", "lut6_layers.cu", "binary_lut6.cu", "stochastic_bn.cu", "no_alloc.cu", "host_io.cu", "losses.cu", "modulation.cu", "conv_lowering.cu", "binary_mode.cu", "frame_buffer.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    os.makedirs(LIB_DIR, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "bbcu_b200.h"))
    if force or _newer(LIB, deps):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-shared"] + srcs + ["-o", LIB]
        subprocess.check_call(cmd)
    return LIB


def build_host_module(force=False):
    """The pybind11 module `binarybrain_b200.core` (C++ host classes in BinaryBrain's style over the C ABI)."""
    import pybind11

    host = os.path.join(HERE, "host")
    src = os.path.join(host, "core_main.cpp")
    if not os.path.exists(src):
        return None
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(HERE, "core" + ext)
    deps = [os.path.join(d, f) for d, _, files in os.walk(host) for f in files] + [LIB, os.path.join(HERE, "..", "include", "bbcu_b200.h")]
    if force or _newer(out, deps):
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", src, "-o", out,
               "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(HERE, "..", "include"),
               "-I/usr/local/cuda/include", "-L" + LIB_DIR, "-lbbcu_b200", "-Wl,-rpath,$ORIGIN/lib",
               "-L/usr/local/cuda/lib64", "-lcudart"]
        subprocess.check_call(cmd)
    return out


def build_all(force=False):
    lib = build_library(force)
    mod = build_host_module(force)
    return lib, mod


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
