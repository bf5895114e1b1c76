"""In-tree build of the two native libraries.

* ``_hsb_kernels.so``  every ``csrc/kernels/*.cu`` and ``csrc/runtime/*.cu`` compiled by nvcc for
  ``sm_100a`` only; exports plain C entry points that the Python ops call through ctypes
  (no torch headers -> seconds to build, cross-compiles on a box without a GPU).
* ``_hsb_core*.so``    the host-side C++ core (distributed-states algebra, reshard planner,
  pipeline schedules, bucket packer, symbolic ints, arena planner, NVML profiler) as a pybind11 module.

Both land inside the package directory so that they travel with the source tree.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
KERNEL_LIB = os.path.join(PKG_DIR, "_hsb_kernels.so")
CORE_LIB = os.path.join(PKG_DIR, "_hsb_core" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
OBJ_DIR = os.path.join(PKG_DIR, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd) + "\n" + proc.stdout)


def find_nvcc() -> str | None:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def kernel_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) + glob.glob(os.path.join(CSRC, "runtime", "*.cu")))


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    srcs = kernel_sources()
    hdrs = glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.h")) + \
        glob.glob(os.path.join(CSRC, "runtime", "*.cuh")) + glob.glob(os.path.join(CSRC, "runtime", "*.h"))
    if not force and _newer(KERNEL_LIB, srcs + hdrs):
        return KERNEL_LIB
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and _newer(o, [s] + hdrs):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "runtime"),
               "-c", s, "-o", o]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + out)
        if verbose:
            print(out)
    _run([nvcc, "-shared", "-o", KERNEL_LIB, *objs, "-lcudart", "-gencode", "arch=compute_100a,code=sm_100a"])
    return KERNEL_LIB


def core_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "core", "*.cc")))


def build_core(force: bool = False) -> str:
    srcs = core_sources()
    hdrs = glob.glob(os.path.join(CSRC, "core", "*.h"))
    if not force and _newer(CORE_LIB, srcs + hdrs):
        return CORE_LIB
    import pybind11
    inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{os.path.join(CSRC, 'core')}"]
    cxx = shutil.which("g++") or "g++"
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and _newer(o, [s] + hdrs):
            continue
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", *inc, "-c", s, "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("g++ failed: " + " ".join(cmd) + "\n" + out)
    _run([cxx, "-shared", "-o", CORE_LIB, *objs, "-ldl", "-lpthread"])
    return CORE_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_core(force)
    build_kernels(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", CORE_LIB, KERNEL_LIB)
