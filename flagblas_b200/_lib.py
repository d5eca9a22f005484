"""Loader of the native code: ``libflagblas_b200.so`` (the C ABI declared in
``include/flagblas_b200.h``) and the pybind11 module ``c_operators`` bound over it.

The operators call through ``c_operators`` (``cop`` below); the ctypes handle ``lib`` exposes
the same C symbols directly (used by tests that exercise the ABI itself).  There is no fallback:
if the native code is missing (and cannot be built because ``nvcc`` / ``g++`` are absent)
importing this module raises, and every operator raises :class:`FlagBlasError` when the library
reports a non-zero status.
"""
import ctypes
import os

from . import build as _build

FB_F32, FB_TF32, FB_F16, FB_BF16 = 0, 1, 2, 3
FB_OK = 0
FB_FP8_E4M3, FB_FP8_E5M2 = 0, 1
FB_F64, FB_C64, FB_C128 = 4, 5, 6


class FlagBlasError(RuntimeError):
    """A non-zero status from the native library (host-side code or device status word)."""

    def __init__(self, status, where=""):
        self.status = status
        text = lib.fb_status_string(status).decode() if lib is not None else "?"
        extra = ""
        if status == -3 and lib is not None:
            extra = " (cudaError %d)" % lib.fb_last_cuda_error()
        super().__init__("flagblas_b200 %s: status %d: %s%s" % (where, status, text, extra))


def _load():
    path = _build.LIB_PATH
    if not _build.up_to_date():
        # No built native code, or one built from other sources than the ones beside it (the binaries are not
        # version controlled): build it now (needs nvcc and g++, not a GPU).
        _build.build()
    handle = ctypes.CDLL(path)
    handle.fb_build_id.restype = ctypes.c_char_p
    handle.fb_build_id.argtypes = []
    if handle.fb_build_id().decode() != _build.source_id():
        raise ImportError("libflagblas_b200.so was built from other sources (build id %s, sources %s); "
                          "run python -m flagblas_b200.build" % (handle.fb_build_id().decode(), _build.source_id()))
    c = ctypes
    i64, f32, vp, sz, i32 = c.c_int64, c.c_float, c.c_void_p, c.c_size_t, c.c_int
    handle.fb_gemm.restype = i32
    handle.fb_gemm.argtypes = [i32, i32, i32, i64, i64, i64, f32, vp, i64, vp, i64, f32, vp, i64, vp, sz, vp]
    handle.fb_gemm_workspace_bytes.restype = sz
    handle.fb_gemm_workspace_bytes.argtypes = [i32, i32, i32, i64, i64, i64, vp, i64, vp, i64]
    handle.fb_gemm_ex.restype = i32
    handle.fb_gemm_ex.argtypes = [i32, i32, i32, i64, i64, i64, c.POINTER(c.c_double), vp, i64, vp, i64,
                                  c.POINTER(c.c_double), vp, i64, vp]
    handle.fb_trmm.restype = i32
    handle.fb_trmm.argtypes = [i32, i32, i32, i32, i32, i64, i64, c.POINTER(c.c_double), vp, i64, vp, i64, vp, i64, vp]
    handle.fb_gemv.restype = i32
    handle.fb_gemv.argtypes = [i32, i32, i64, i64, f32, vp, i64, vp, i64, f32, vp, i64, vp, sz, vp]
    handle.fb_gemv_workspace_bytes.restype = sz
    handle.fb_gemv_workspace_bytes.argtypes = [i32, i32, i64, i64]
    handle.fb_gemv_fp8.restype = i32
    handle.fb_gemv_fp8.argtypes = [i32, i32, i32, i64, i64, f32, vp, i64, vp, i64, f32, vp, i64, vp, sz, vp]
    handle.fb_gemv_fp8_workspace_bytes.restype = sz
    handle.fb_gemv_fp8_workspace_bytes.argtypes = [i64, i64]
    handle.fb_group_gemm.restype = i32
    handle.fb_group_gemm.argtypes = [i32, i32] + [vp] * 10 + [i32, i64, i64, i64, f32, f32, vp, sz, vp]
    handle.fb_group_gemm_prepare.restype = i32
    handle.fb_group_gemm_prepare.argtypes = [i32, i32] + [vp] * 10 + [i32, i64, i64, i64, vp, sz, vp]
    handle.fb_group_gemm_run.restype = i32
    handle.fb_group_gemm_run.argtypes = [i32, i32, i32, i64, i64, i64, f32, f32, vp, sz, vp]
    handle.fb_group_gemm_no_alloc.restype = i32
    handle.fb_group_gemm_no_alloc.argtypes = [i32, i32] + [vp] * 10 + [i32, i64, i64, i64, f32, f32, vp]
    handle.fb_no_alloc_max_groups.restype = i32
    handle.fb_no_alloc_max_groups.argtypes = []
    handle.fb_group_mm.restype = i32
    handle.fb_group_mm.argtypes = [i32, i32, vp, i64, vp, i64, i64, vp, i64, vp, i32, i64, i64, vp, sz, vp]
    handle.fb_group_workspace_bytes.restype = sz
    handle.fb_group_workspace_bytes.argtypes = [i32]
    handle.fb_group_min_workspace_bytes.restype = sz
    handle.fb_group_min_workspace_bytes.argtypes = [i32]
    handle.fb_status_string.restype = c.c_char_p
    handle.fb_status_string.argtypes = [i32]
    handle.fb_device_status.restype = i32
    handle.fb_device_status.argtypes = [i32]
    handle.fb_last_cuda_error.restype = i32
    handle.fb_last_cuda_error.argtypes = []
    handle.fb_sm_count.restype = i32
    handle.fb_sm_count.argtypes = []
    handle.fb_reload_env.restype = None
    handle.fb_reload_env.argtypes = []
    handle.fb_debug_set_profile_buffer.restype = None
    handle.fb_debug_set_profile_buffer.argtypes = [vp]
    handle.fb_selftest_bounded_wait.restype = i32
    handle.fb_selftest_bounded_wait.argtypes = [i64, vp]
    return handle


lib = None
lib = _load()
from . import c_operators as cop  # noqa: E402  (pybind11 module; links against the library loaded above)

# Every symbol include/flagblas_b200.h declares; tests check the library exports them all.
EXPORTED_SYMBOLS = (
    "fb_gemm",
    "fb_gemm_workspace_bytes",
    "fb_gemm_ex",
    "fb_trmm",
    "fb_gemv",
    "fb_gemv_workspace_bytes",
    "fb_gemv_fp8",
    "fb_gemv_fp8_workspace_bytes",
    "fb_group_gemm",
    "fb_group_mm",
    "fb_group_gemm_no_alloc",
    "fb_group_gemm_prepare",
    "fb_group_gemm_run",
    "fb_no_alloc_max_groups",
    "fb_group_workspace_bytes",
    "fb_group_min_workspace_bytes",
    "fb_status_string",
    "fb_device_status",
    "fb_last_cuda_error",
    "fb_sm_count",
    "fb_reload_env",
    "fb_build_id",
    "fb_selftest_bounded_wait",
    "fb_debug_set_profile_buffer",
)


# ---------------------------------------------------------------- per-call host plumbing
# Kept as short as possible: for small problems the host side of a call costs more than the kernel.
_scratch_cache = {}


def enter(device):
    """Make ``device`` current if it is not; returns (raw current stream of it, device to restore or -1)."""
    import torch

    idx = device.index
    if idx is None:
        idx = torch.cuda.current_device()
    cur = torch._C._cuda_getDevice()
    prev = -1
    if cur != idx:
        torch.cuda.set_device(idx)
        prev = cur
    return torch._C._cuda_getCurrentRawStream(idx), prev


def leave(prev):
    if prev >= 0:
        import torch

        torch.cuda.set_device(prev)


def scratch(device, stream, nbytes):
    """Address of at least ``nbytes`` of device scratch tied to (device, stream).

    One buffer per (device, stream) is kept and grown on demand: calls on one stream run in order, so
    the next call may overwrite what the previous one left -- exactly the reuse rule of the C ABI's
    workspace arguments.  Costs at most the largest request per stream for the life of the process.
    """
    if nbytes == 0:
        return 0
    key = (device.index, stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        import torch

        size = 1 << max(16, (nbytes - 1).bit_length())
        buf = torch.empty(size, dtype=torch.uint8, device=device)
        _scratch_cache[key] = buf
    return buf.data_ptr()


def check(status, where=""):
    if status != FB_OK:
        raise FlagBlasError(status, where)


def device_status(reset=True):
    """Synchronise and return the device status word (0 = healthy)."""
    return cop.device_status(1 if reset else 0)


def reload_env():
    """Have the library read its ``FLAGBLAS_B200_*`` switches again (it reads the environment once per process)."""
    cop.reload_env()
