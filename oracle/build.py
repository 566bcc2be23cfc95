"""Build recipe for the CPU oracle (test infrastructure, never the product path).

Two artefacts:

* ``oracle/_build/libbcpnn_oracle.so`` -- our own plain-C restatement
  (``bcpnn_oracle.c``), strict IEEE arithmetic, OpenMP.
* ``oracle/_ref/_bcpnn_kernels_openmp_internal<EXT_SUFFIX>`` -- StreamBrain's own
  OpenMP kernel module, compiled straight from the reference checkout's
  ``BCPNN/backend/_kernels/kernels_openmp_internal.cc`` with the flags its
  ``CMakeLists.txt:24,40-41`` uses (``-O3 -march=native -ffast-math -fopenmp``).
  Only attempted when a reference checkout is present (``SBB_REFERENCE_ROOT`` or
  a directory ``reference`` beside this repository); the source file is compiled where it lies and nothing
  but the resulting shared object is written.  ``<cblas.h>`` is our own shim
  header and the BLAS is the OpenBLAS shared object bundled in the SciPy (or
  OpenCV) wheel.  The reference's cmake build is not run.

Run ``python oracle/build.py`` or call :func:`build_all`.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_LIB = os.path.join(BUILD_DIR, "libbcpnn_oracle.so")
REF_MODULE_NAME = "_bcpnn_kernels_openmp_internal"
REF_KERNEL_SOURCE = os.path.join("BCPNN", "backend", "_kernels", "kernels_openmp_internal.cc")


def reference_root() -> str | None:
    """A StreamBrain checkout: ``SBB_REFERENCE_ROOT``, else a directory ``reference`` beside this repository."""
    root = os.environ.get("SBB_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return root if os.path.isfile(os.path.join(root, REF_KERNEL_SOURCE)) else None


# The reference builds with -march=native (CMakeLists.txt:40-41).  The module is
# compiled on one machine and run on another, so two portable ISA levels are
# built instead and the loader picks the widest one the running CPU supports.
REF_ISA_LEVELS = ("x86-64-v4", "x86-64-v3")
_V4_FLAGS = {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"}


def cpu_isa_level() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return "x86-64-v4" if _V4_FLAGS <= set(line.split(":", 1)[1].split()) else "x86-64-v3"
    except OSError:
        pass
    return "x86-64-v3"


def ref_module_path(isa: str | None = None) -> str:
    isa = isa or cpu_isa_level()
    return os.path.join(REF_DIR, isa, REF_MODULE_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def build_oracle(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "bcpnn_oracle.c"), os.path.join(HERE, "bcpnn_oracle_impl.h")]
    if not force and _newer(ORACLE_LIB, srcs):
        return ORACLE_LIB
    os.makedirs(BUILD_DIR, exist_ok=True)
    _run(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
          "-fPIC", "-shared", "-std=c11", "-o", ORACLE_LIB, srcs[0], "-lm"])
    return ORACLE_LIB


def find_openblas() -> tuple[str, bool] | None:
    """Return (path, uses_scipy_prefix) of a wheel-bundled OpenBLAS, if any."""
    for sp in [p for p in sys.path if p.endswith("site-packages")] + [sysconfig.get_paths()["purelib"]]:
        hits = sorted(glob.glob(os.path.join(sp, "scipy.libs", "libscipy_openblas*.so")))
        if hits:
            return hits[0], True
        hits = sorted(glob.glob(os.path.join(sp, "opencv_python_headless.libs", "libopenblasp*.so")))
        if hits:
            return hits[0], False
    return None


def build_reference(force: bool = False) -> str | None:
    """Compile the reference's OpenMP kernel module into oracle/_ref/.

    Returns the module path, or None when no reference checkout is present and no
    previously built module exists (the GPU box only ever uses the prebuilt file).
    """
    root = reference_root()
    if root is None:
        out = ref_module_path()
        return out if os.path.exists(out) else None
    for isa in REF_ISA_LEVELS:
        _build_reference_isa(root, isa, force)
    return ref_module_path()


def _build_reference_isa(root: str, isa: str, force: bool) -> None:
    out = ref_module_path(isa)
    src = os.path.join(root, REF_KERNEL_SOURCE)
    shim = os.path.join(HERE, "shim", "cblas.h")
    if not force and _newer(out, [src, shim]):
        return
    blas = find_openblas()
    if blas is None:
        raise RuntimeError("no wheel-bundled OpenBLAS found; the reference module cannot be linked")
    blas_path, scipy_prefix = blas
    import pybind11

    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = ["g++", "-O3", "-march=" + isa, "-ffast-math", "-fopenmp", "-fPIC", "-shared", "-std=c++17",
           "-Wno-register", "-w",
           "-I" + os.path.join(HERE, "shim"), "-I" + sysconfig.get_paths()["include"],
           "-I" + pybind11.get_include()]
    if scipy_prefix:
        cmd.append("-DSBB_CBLAS_SCIPY_PREFIX")
    cmd += ["-o", out, src, blas_path,
            "-Wl,-rpath," + os.path.dirname(blas_path)]
    _run(cmd)
    with open(os.path.join(os.path.dirname(out), "BUILD_INFO.txt"), "w") as f:
        f.write("source: %s (compiled in place, not copied)\nblas: %s\ncmd: %s\n" %
                (REF_KERNEL_SOURCE, os.path.basename(blas_path), " ".join(cmd)))


# The reference's own kernel test (a script that compares a kernel module with its NumPy kernels) and the two
# modules it imports.  They are staged, unmodified, beside the compiled module so that the GPU box -- which has
# no reference checkout -- can run that test against this repository's kernel module.  The directory is
# git-ignored: nothing of the reference enters the history.
CONTRACT_DIR = os.path.join(REF_DIR, "contract")
CONTRACT_FILES = ("test_openmp.py", "kernels_numpy.py", "kernels_openmp.py")


def stage_reference_contract() -> str | None:
    root = reference_root()
    if root is None:
        return CONTRACT_DIR if os.path.exists(os.path.join(CONTRACT_DIR, CONTRACT_FILES[0])) else None
    import shutil
    os.makedirs(CONTRACT_DIR, exist_ok=True)
    for name in CONTRACT_FILES:
        shutil.copyfile(os.path.join(root, "BCPNN", "backend", "_kernels", name), os.path.join(CONTRACT_DIR, name))
    return CONTRACT_DIR


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "reference": build_reference(force),
            "contract": stage_reference_contract()}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
