"""Builds libsbb200.so in-tree with nvcc for sm_100a.

    python -m streambrain_b200.build [--force] [--verbose]

The shared object is written next to this file (it is git-ignored but travels
with a snapshot of the tree), so importing the package never needs a compiler on
the machine that runs it.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsbb200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--shared", "-cudart", "static"]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list[str]:
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(s) <= t for s in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libsbb200.so must be built where the CUDA toolkit is installed")
    # linked under another name and moved into place: an interrupted build never leaves a torn library behind
    tmp = LIB + ".%d.tmp" % os.getpid()
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-I" + INCLUDE, "-o", tmp] + sources()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed:\n%s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))
    os.replace(tmp, LIB)
    if verbose:
        print(proc.stderr)
    return LIB


PYBIND_SRC = os.path.join(HERE, "pybind", "bcpnn_kernels_b200_internal.cpp")


def pybind_module_path() -> str:
    import sysconfig
    return os.path.join(HERE, "_bcpnn_kernels_b200_internal" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pybind(force: bool = False) -> str | None:
    """The pybind11 kernel module with the reference's function names, linked against libsbb200.so
    (found at run time next to the module).  Returns None where pybind11 is not installed."""
    import sysconfig
    try:
        import pybind11
    except ImportError:
        return None
    out = pybind_module_path()
    deps = [PYBIND_SRC, LIB] + glob.glob(os.path.join(INCLUDE, "*.h"))
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-I" + INCLUDE,
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-o", out, PYBIND_SRC,
           "-L" + HERE, "-l:libsbb200.so", "-Wl,-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("g++ failed:\n%s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_pybind(force="--force" in sys.argv))
