"""BLAS enum values, as exported by the reference (``src/flag_blas/ops/level2/_constants.py``)."""
CUBLAS_OP_N = 0
CUBLAS_OP_T = 1
CUBLAS_OP_C = 2
