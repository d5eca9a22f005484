"""BLAS enum values, as exported by the reference (``src/flag_blas/ops/level2/_constants.py``)."""
CUBLAS_OP_N = 0
CUBLAS_OP_T = 1
CUBLAS_OP_C = 2
CUBLAS_FILL_MODE_LOWER = 0
CUBLAS_FILL_MODE_UPPER = 1
CUBLAS_DIAG_NON_UNIT = 0
CUBLAS_DIAG_UNIT = 1
CUBLAS_SIDE_LEFT = 0     # (defined in the reference's ops/level3/trmm.py:25-26)
CUBLAS_SIDE_RIGHT = 1
