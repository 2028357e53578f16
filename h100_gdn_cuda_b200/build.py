"""Builds libgdn_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m h100_gdn_cuda_b200.build [--force]

The shared object lands in h100_gdn_cuda_b200/lib/ and is what the Python layer loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libgdn_b200.so")
SOURCES = ["gdn_b200.cu", "gdn_prefill.cu", "gdn_jit.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]


def nvcc_path() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_HOME_PATH"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _deps_mtime() -> float:
    newest = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    newest = max(newest, os.path.getmtime(os.path.join(PKG, "..", "include", "gdn_b200.h")))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = nvcc_path()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    os.replace(LIB + ".tmp", LIB)
    return LIB


EXT_DIR = os.path.join(CSRC, "torch_ext")


def ext_path() -> str:
    import sysconfig
    return os.path.join(PKG, "gdn_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_ext(force: bool = False) -> str:
    """Builds the pybind11/torch extension `gdn_cuda` (C++ host layer over the C ABI) in-tree."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    lib = build(force=False)
    out = ext_path()
    srcs = [os.path.join(EXT_DIR, f) for f in ("gdn_api.cpp", "python_api.cpp")]
    newest = max(os.path.getmtime(f) for f in srcs + [os.path.join(EXT_DIR, "gdn_api.hpp"),
                                                       os.path.join(PKG, "..", "include", "gdn_b200.h")])
    if not force and os.path.exists(out) and os.path.getmtime(out) >= newest:
        return out
    inc = cpp_extension.include_paths("cuda") if hasattr(cpp_extension, "include_paths") else []
    try:
        inc = cpp_extension.include_paths(device_type="cuda")
    except TypeError:
        inc = cpp_extension.include_paths(True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.path.dirname(os.path.dirname(nvcc_path()))
    objs = []

    def cc(src):
        obj = os.path.join(OBJDIR, os.path.basename(src).replace(".cpp", ".ext.o"))
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=gdn_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
               "-I", os.path.join(PKG, "..", "include"), "-I", sysconfig.get_paths()["include"],
               "-I", os.path.join(cuda_home, "include")]
        for i in inc:
            cmd += ["-isystem", i]
        cmd += ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed for %s:\n%s" % (src, r.stderr[-4000:]))
        return obj

    os.makedirs(OBJDIR, exist_ok=True)
    with ThreadPoolExecutor(max_workers=2) as ex:
        objs = list(ex.map(cc, srcs))
    cmd = ["g++", "-shared", "-o", out + ".tmp", *objs, "-L", tlib, "-L", LIBDIR, "-lgdn_b200", "-ltorch", "-ltorch_cpu",
           "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python", "-L", os.path.join(cuda_home, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath," + tlib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s" % r.stderr[-4000:])
    os.replace(out + ".tmp", out)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--ext" in sys.argv:
        print(build_ext(force="--force" in sys.argv))
