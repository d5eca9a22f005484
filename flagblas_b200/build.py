"""Build recipe for the native library: one nvcc invocation, sm_100a only.

The shared object is written next to this file (``libflagblas_b200.so``) so that
it is found in-tree by :mod:`flagblas_b200._lib`.  ``python -m flagblas_b200.build``
rebuilds it.
"""
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflagblas_b200.so")
_SRC = os.path.join(_HERE, "csrc", "flagblas_b200.cu")
_DEPS = sorted(
    os.path.join(_HERE, "csrc", f) for f in os.listdir(os.path.join(_HERE, "csrc")) if f.endswith((".cu", ".cuh"))
) + [os.path.join(os.path.dirname(_HERE), "include", "flagblas_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return exe


EXT_SUFFIX = __import__("sysconfig").get_config_var("EXT_SUFFIX") or ".so"
EXT_PATH = os.path.join(_HERE, "c_operators" + EXT_SUFFIX)
_EXT_SRC = os.path.join(_HERE, "csrc", "c_operators.cpp")


def build_extension(force=False):
    """Compile the pybind11 module ``flagblas_b200.c_operators`` (g++; links against the library)."""
    deps = [_EXT_SRC, os.path.join(os.path.dirname(_HERE), "include", "flagblas_b200.h"), LIB_PATH]
    if not force and os.path.exists(EXT_PATH) and all(os.path.getmtime(d) <= os.path.getmtime(EXT_PATH) for d in deps):
        return EXT_PATH
    import sysconfig

    import pybind11

    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise RuntimeError("g++ not found; the pybind11 module cannot be built")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], _EXT_SRC,
           "-L" + _HERE, "-lflagblas_b200", "-Wl,-rpath,$ORIGIN", "-o", EXT_PATH]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return EXT_PATH


def up_to_date():
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    return all(not os.path.exists(d) or os.path.getmtime(d) <= t for d in _DEPS)


def build(force=False, verbose=False):
    """Compile ``csrc/flagblas_b200.cu`` into ``libflagblas_b200.so`` (no GPU needed)."""
    if not force and up_to_date():
        build_extension()
        return LIB_PATH
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH, _SRC]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    build_extension(force=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
