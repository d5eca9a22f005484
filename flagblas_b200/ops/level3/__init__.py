from .gemm import bfgemm, hgemm, sgemm, tf32gemm
from .trmm import ctrmm, dtrmm, strmm, ztrmm
from .xgemm import cgemm, dgemm, zgemm
from .group_gemm import group_bfgemm, group_gemm, group_hgemm, group_mm, group_tf32gemm

__all__ = [
    "sgemm", "hgemm", "bfgemm", "tf32gemm",
    "group_bfgemm", "group_hgemm", "group_tf32gemm", "group_mm", "group_gemm",
    "dgemm", "cgemm", "zgemm",
    "strmm", "dtrmm", "ctrmm", "ztrmm",
]
