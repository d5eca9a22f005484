"""flagblas_b200 -- B200 (sm_100a) implementation of FlagBLAS's GEMM family.

Exports the same operator names as ``flag_blas`` for this path (``sgemm``, ``hgemm``,
``bfgemm``, ``group_bfgemm``, ``group_hgemm``, ``group_tf32gemm``, ``group_mm``) plus the
dense ``tf32gemm`` and the ``group_gemm`` convenience wrapper, the ``CUBLAS_OP_*``
constants, ``device`` / ``vendor_name``, ``testing`` and ``runtime.device``, the matrix-vector operators
``sgemv`` / ``hgemv`` / ``bfgemv``, and the ``enable`` / ``only_enable`` / ``use_blas`` registration entry points
that put the kernels behind ``torch.mm`` and friends.
Importing it loads the native library; there is no CPU or eager fallback.
"""
from . import runtime, testing  # noqa: F401
from . import _lib
from .ops import *  # noqa: F401,F403
from .ops import __all__ as _ops_all
from ._lib import FlagBlasError, device_status, reload_env  # noqa: F401

# ``flag_blas.c_operators`` is the name the reference reserves for a compiled extension
# (src/flag_blas/config.py:35-41); here it is the pybind11 module over the C ABI.
from . import c_operators  # noqa: E402,F401
from . import host  # noqa: E402,F401
from .ops.level3.group_gemm import GroupPlan, group_prepare  # noqa: E402,F401
from .aten import all_registered_keys, all_registered_ops, enable, only_enable, use_blas  # noqa: E402,F401

device = runtime.device.name
vendor_name = runtime.device.vendor_name
__version__ = "0.1.0"

__all__ = list(_ops_all) + ["runtime", "testing", "device", "vendor_name", "c_operators", "FlagBlasError",
                            "device_status", "reload_env", "host", "group_prepare", "GroupPlan", "enable", "only_enable", "use_blas", "all_registered_ops",
                            "all_registered_keys"]
