"""Dense GEMM in double and complex precision: ``dgemm``, ``cgemm``, ``zgemm``.

Same call signature and semantics as the reference operators (``src/flag_blas/ops/level3/dgemm.py:160-208``,
``cgemm.py:192-254``, ``zgemm.py:192-254``):

    X(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None

row-major, in place on ``C``; the complex flavours also accept ``CUBLAS_OP_C`` and complex ``alpha`` /
``beta``.  The arithmetic runs in the native library (``fb_gemm_ex``: IEEE FMAs on the CUDA cores in the
operand's own precision -- the reference's ``cgemm`` forms its products from split TF32 dots instead, so the
two agree to single-precision accuracy, not bit for bit).
"""
import torch

from ... import _lib
from .._constants import CUBLAS_OP_C, CUBLAS_OP_N, CUBLAS_OP_T

_cop = _lib.cop


def _parts(v):
    v = v.item() if isinstance(v, torch.Tensor) else v
    v = complex(v)
    return float(v.real), float(v.imag)


def _required_numel(rows, cols, ld):
    return 0 if rows == 0 or cols == 0 else (rows - 1) * ld + cols


def _xgemm(code, dtype, name, ops_allowed, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    # argument checks of the reference (dgemm.py:109-157, cgemm.py:39-100)
    assert A.is_contiguous()
    assert B.is_contiguous()
    assert C.is_contiguous()
    assert A.dtype == dtype
    assert B.dtype == dtype
    assert C.dtype == dtype
    assert A.device == B.device == C.device
    assert transa in ops_allowed
    assert transb in ops_allowed
    if transa == CUBLAS_OP_N:
        if m > 0 and k > 0:
            assert lda >= k
        assert A.numel() >= _required_numel(m, k, lda)
    else:
        if m > 0 and k > 0:
            assert lda >= m
        assert A.numel() >= _required_numel(k, m, lda)
    if transb == CUBLAS_OP_N:
        if n > 0 and k > 0:
            assert ldb >= n
        assert B.numel() >= _required_numel(k, n, ldb)
    else:
        if n > 0 and k > 0:
            assert ldb >= k
        assert B.numel() >= _required_numel(n, k, ldb)
    if m > 0 and n > 0:
        assert ldc >= n
    assert C.numel() >= _required_numel(m, n, ldc)
    if not C.is_cuda:
        raise RuntimeError("flagblas_b200.%s: tensors must live on a CUDA device (there is no CPU path)" % name)

    ar, ai = _parts(alpha)
    br, bi = _parts(beta)
    if not dtype.is_complex:
        ai = bi = 0.0
    stream, prev = _lib.enter(C.device)
    try:
        if m == 0 or n == 0 or k == 0 or (ar == 0.0 and ai == 0.0):
            # the reference scales *every* element of C here (dgemm.py:180-185): a (1 x numel) block, k = 0
            numel = C.numel()
            status = 0
            if numel and not (br == 1.0 and bi == 0.0):
                status = _cop.gemm_ex(code, 0, 0, 1, numel, 0, 0.0, 0.0, 0, 1, 0, numel, br, bi, C.data_ptr(), numel,
                                      stream)
        else:
            status = _cop.gemm_ex(code, transa, transb, m, n, k, ar, ai, A.data_ptr(), lda, B.data_ptr(), ldb, br, bi,
                                  C.data_ptr(), ldc, stream)
    finally:
        _lib.leave(prev)
    if status:
        _lib.check(status, name)


def dgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """fp64 GEMM (reference: ops/level3/dgemm.py:160-208)."""
    _xgemm(_lib.FB_F64, torch.float64, "dgemm", (CUBLAS_OP_N, CUBLAS_OP_T), transa, transb, m, n, k, alpha, A, lda, B,
           ldb, beta, C, ldc)


def cgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """complex64 GEMM, op in {N, T, C} (reference: ops/level3/cgemm.py:192-254)."""
    _xgemm(_lib.FB_C64, torch.complex64, "cgemm", (CUBLAS_OP_N, CUBLAS_OP_T, CUBLAS_OP_C), transa, transb, m, n, k,
           alpha, A, lda, B, ldb, beta, C, ldc)


def zgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """complex128 GEMM, op in {N, T, C} (reference: ops/level3/zgemm.py:192-254)."""
    _xgemm(_lib.FB_C128, torch.complex128, "zgemm", (CUBLAS_OP_N, CUBLAS_OP_T, CUBLAS_OP_C), transa, transb, m, n, k,
           alpha, A, lda, B, ldb, beta, C, ldc)
