"""In-tree build of the native parts (no setuptools, no JIT cache):

* ``ops3d_b200/libfda_b200.so``  -- CUDA kernels + C ABI (``include/fda_b200.h``), nvcc for sm_100a only;
  depends on nothing but the CUDA runtime.
* ``ops3d_b200/_C*.so``          -- thin torch/pybind11 binding (host C++ only) linked against it.

``python -m ops3d_b200.build`` builds whatever is out of date; ``--force`` rebuilds.
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libfda_b200.so")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
EXT = os.path.join(PKG, "_C" + EXT_SUFFIX)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",  # CUDA runtime linked statically: the library needs only the driver
]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    srcs.append(os.path.join(ROOT, "include", "fda_b200.h"))
    if not force and _newer(LIB, srcs):
        return LIB
    units = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    # one nvcc per translation unit, side by side, then one link
    objdir = os.path.join(PKG, "_obj")
    os.makedirs(objdir, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]
    extra = os.environ.get("FDA_NVCC_EXTRA", "").split()  # e.g. -DFDA_BWD_MIN_BLOCKS=3 for experiments
    objs = [os.path.join(objdir, os.path.basename(u)[:-3] + ".o") for u in units]
    procs = []
    for u, o in zip(units, objs):
        cmd = [_nvcc(), *compile_flags, *extra, "-c", u, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, proc in procs:
        if proc.wait() != 0:
            raise subprocess.CalledProcessError(proc.returncode, cmd)
    _run([_nvcc(), *NVCC_FLAGS, *objs, "-o", LIB], verbose)
    return LIB


def build_binding(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "binding.cpp")
    if not force and _newer(EXT, [src, os.path.join(ROOT, "include", "fda_b200.h"), LIB]):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdirs = ce.library_paths("cuda")
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall",
        "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *inc, src, "-o", EXT,
        f"-L{PKG}", "-lfda_b200", "-Wl,-rpath,$ORIGIN",
    ]
    for d in libdirs:
        cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(cmd, verbose)
    return EXT


def build_all(force: bool = False, verbose: bool = False):
    return build_library(force, verbose), build_binding(force, verbose)


if __name__ == "__main__":
    out = build_all(force="--force" in sys.argv, verbose=True)
    print("built:", *out)
