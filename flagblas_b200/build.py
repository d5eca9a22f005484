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

ID_PATH = LIB_PATH + ".buildid"


def source_id():
    """Hash of every source the library is compiled from (and of the flags): the library carries it
    (``fb_build_id()``) so that a binary built from other sources is never loaded silently."""
    import hashlib

    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for path in _DEPS + [_EXT_SRC]:
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    return h.hexdigest()[:32]


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
    """True when the built library and extension were made from the sources as they are now."""
    if not (os.path.exists(LIB_PATH) and os.path.exists(EXT_PATH) and os.path.exists(ID_PATH)):
        return False
    with open(ID_PATH) as f:
        return f.read().strip() == source_id()


def build(force=False, verbose=False):
    """Compile ``csrc/flagblas_b200.cu`` into ``libflagblas_b200.so`` (no GPU needed)."""
    if not force and up_to_date():
        return LIB_PATH
    sid = source_id()
    if os.path.exists(ID_PATH):
        os.remove(ID_PATH)
    cmd = ([_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) +
           ['-DFB_BUILD_ID="%s"' % sid, "-o", LIB_PATH, _SRC])
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    build_extension(force=True)
    with open(ID_PATH, "w") as f:
        f.write(sid + "\n")
    return LIB_PATH


if __name__ == "__main__":
    # (importing the package has already rebuilt a stale binary; -f compiles again regardless)
    print(build(force="-f" in sys.argv or "-v" in sys.argv, verbose="-v" in sys.argv))
