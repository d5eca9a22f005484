"""Triangular matrix products: ``strmm``, ``dtrmm``, ``ctrmm``, ``ztrmm``.

Same call signature and semantics as the reference operators (``src/flag_blas/ops/level3/trmm.py:2095-2231``,
``2234-2329``, ``3161-3292``, ``4743-4939``):

    X(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc) -> None

row-major; ``side = LEFT``: ``C = alpha * op(tri(A)) @ B`` with ``A`` ``[m, m]``; ``side = RIGHT``:
``C = alpha * B @ op(tri(A))`` with ``A`` ``[n, n]``; only the ``uplo`` triangle of ``A`` is read and
``diag = UNIT`` reads its diagonal as 1.  Out of place: the result goes to ``C`` (``B`` may be the same tensor).
The arithmetic runs in the native library (``fb_trmm``).
"""
import torch

from ... import _lib
from .._constants import (CUBLAS_DIAG_NON_UNIT, CUBLAS_DIAG_UNIT, CUBLAS_FILL_MODE_LOWER, CUBLAS_FILL_MODE_UPPER,
                          CUBLAS_OP_C, CUBLAS_OP_N, CUBLAS_OP_T, CUBLAS_SIDE_LEFT, CUBLAS_SIDE_RIGHT)

_cop = _lib.cop


def _check_trmm(A, B, C, side, uplo, trans, diag, m, n, lda, ldb, ldc, complex_ok):
    # the reference's checks (trmm.py:2061-2080)
    assert A.is_contiguous()
    assert B.is_contiguous()
    assert C.is_contiguous()
    assert A.device == B.device == C.device
    assert side in (CUBLAS_SIDE_LEFT, CUBLAS_SIDE_RIGHT)
    assert uplo in (CUBLAS_FILL_MODE_LOWER, CUBLAS_FILL_MODE_UPPER)
    if complex_ok:
        assert trans in (CUBLAS_OP_N, CUBLAS_OP_T, CUBLAS_OP_C)
    else:
        assert trans in (CUBLAS_OP_N, CUBLAS_OP_T)
    assert diag in (CUBLAS_DIAG_NON_UNIT, CUBLAS_DIAG_UNIT)
    assert m >= 0 and n >= 0
    k = m if side == CUBLAS_SIDE_LEFT else n
    assert lda >= max(1, k)
    assert ldb >= max(1, n)
    assert ldc >= max(1, n)
    assert A.numel() >= max(1, k) * lda
    assert B.numel() >= max(1, m) * ldb
    assert C.numel() >= max(1, m) * ldc


def _trmm(code, dtype, name, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc):
    assert A.dtype == dtype == B.dtype == C.dtype
    _check_trmm(A, B, C, side, uplo, trans, diag, m, n, lda, ldb, ldc, dtype.is_complex)
    if not C.is_cuda:
        raise RuntimeError("flagblas_b200.%s: tensors must live on a CUDA device (there is no CPU path)" % name)
    alpha = alpha.item() if isinstance(alpha, torch.Tensor) else alpha
    alpha = complex(alpha)
    ar, ai = float(alpha.real), (float(alpha.imag) if dtype.is_complex else 0.0)
    if m == 0 or n == 0:
        return
    # in-place use: the product reads every row (left) / column (right) of B for each output element
    b_work = B.clone() if (B.data_ptr() == C.data_ptr() and not (ar == 0.0 and ai == 0.0)) else B
    stream, prev = _lib.enter(C.device)
    try:
        status = _cop.trmm(code, side, uplo, trans, diag, m, n, ar, ai, A.data_ptr(), lda, b_work.data_ptr(), ldb,
                           C.data_ptr(), ldc, stream)
    finally:
        _lib.leave(prev)
    if status:
        _lib.check(status, name)


def strmm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc) -> None:
    """fp32 triangular product (reference: ops/level3/trmm.py:2095-2231)."""
    _trmm(_lib.FB_F32, torch.float32, "strmm", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)


def dtrmm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc) -> None:
    """fp64 triangular product (reference: ops/level3/trmm.py:2234-2329)."""
    _trmm(_lib.FB_F64, torch.float64, "dtrmm", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)


def ctrmm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc) -> None:
    """complex64 triangular product, op in {N, T, C} (reference: ops/level3/trmm.py:3161-3292)."""
    _trmm(_lib.FB_C64, torch.complex64, "ctrmm", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)


def ztrmm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc) -> None:
    """complex128 triangular product, op in {N, T, C} (reference: ops/level3/trmm.py:4743-4939)."""
    _trmm(_lib.FB_C128, torch.complex128, "ztrmm", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)
