"""Drop-in alias: ``import flag_blas`` resolves to the B200 back end for the GEMM path.

Keeps the reference's import spellings working (``flag_blas.hgemm``,
``from flag_blas.ops import CUBLAS_OP_N``, ``flag_blas.testing.assert_close``,
``flag_blas.runtime.device.support_bf16``)."""
import sys

import flagblas_b200 as _impl
from flagblas_b200 import *  # noqa: F401,F403
from flagblas_b200 import c_operators, device, ops, runtime, testing, vendor_name, __version__  # noqa: F401

sys.modules[__name__ + ".ops"] = ops
sys.modules[__name__ + ".ops.level3"] = ops.level3
sys.modules[__name__ + ".ops.level2"] = ops.level2
sys.modules[__name__ + ".testing"] = testing
sys.modules[__name__ + ".runtime"] = runtime
