"""Operator exports: the GEMM names and BLAS constants of ``flag_blas.ops``
(reference: ``src/flag_blas/ops/__init__.py:35-52,75-94,151-158``)."""
from ._constants import (CUBLAS_DIAG_NON_UNIT, CUBLAS_DIAG_UNIT, CUBLAS_FILL_MODE_LOWER, CUBLAS_FILL_MODE_UPPER,
                         CUBLAS_OP_C, CUBLAS_OP_N, CUBLAS_OP_T, CUBLAS_SIDE_LEFT, CUBLAS_SIDE_RIGHT)
from .level2 import bfgemv, fp8_gemv, hgemv, sgemv
from .level3 import (bfgemm, cgemm, ctrmm, dgemm, dtrmm, strmm, zgemm, ztrmm, group_bfgemm, group_gemm, group_hgemm, group_mm, group_tf32gemm, hgemm, sgemm,
                     tf32gemm)

__all__ = [
    "CUBLAS_OP_N", "CUBLAS_OP_T", "CUBLAS_OP_C",
    "CUBLAS_FILL_MODE_LOWER", "CUBLAS_FILL_MODE_UPPER", "CUBLAS_DIAG_NON_UNIT", "CUBLAS_DIAG_UNIT",
    "CUBLAS_SIDE_LEFT", "CUBLAS_SIDE_RIGHT",
    "sgemm", "hgemm", "bfgemm", "tf32gemm",
    "group_bfgemm", "group_hgemm", "group_tf32gemm", "group_mm", "group_gemm",
    "sgemv", "hgemv", "bfgemv", "fp8_gemv",
    "dgemm", "cgemm", "zgemm",
    "strmm", "dtrmm", "ctrmm", "ztrmm",
]
