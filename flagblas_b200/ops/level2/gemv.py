"""Matrix-vector operators: ``sgemv``, ``hgemv``, ``bfgemv``, ``fp8_gemv``.

Same call signature and semantics as the reference operators
(``src/flag_blas/ops/level2/gemv.py:2285-2375, 2814-2926, 2929-3041``):

    X(trans, m, n, alpha, A, lda, x, incx, beta, y, incy) -> None

``A`` row-major ``[m, lda >= n]``; ``trans = N``: ``y[m] = alpha*A@x[n] + beta*y``;
``trans = T``: ``y[n] = alpha*A.T@x[m] + beta*y``; ``x`` and ``y`` strided by ``incx``/``incy``;
in place on ``y``.  Products and sums are fp32 for all three types; the result is rounded once.

The arithmetic runs in the native library (``fb_gemv``); this module validates arguments the way
the reference does and hands over raw addresses and the current CUDA stream.
"""
import torch

from ... import _lib
from .._constants import CUBLAS_OP_N, CUBLAS_OP_T

_cop = _lib.cop


def _scalar(v):
    return v.item() if isinstance(v, torch.Tensor) else float(v)


def _call(code, name, trans, m, n, alpha, a_ptr, lda, x_ptr, incx, beta, y_ptr, incy, device):
    stream, prev = _lib.enter(device)
    try:
        # fp32 partial sums of a split reduced dimension live in per-stream scratch
        ws_bytes = _cop.gemv_workspace_bytes(code, trans, m, n) if alpha != 0.0 else 0
        ws_ptr = _lib.scratch(device, stream, ws_bytes)
        status = _cop.gemv(code, trans, m, n, alpha, a_ptr, lda, x_ptr, incx, beta, y_ptr, incy, ws_ptr, ws_bytes,
                           stream)
    finally:
        _lib.leave(prev)
    if status:
        _lib.check(status, name)


def _gemv(code, dtype, name, trans, m, n, alpha, A, lda, x, incx, beta, y, incy):
    assert A.is_contiguous()
    assert x.is_contiguous()
    assert y.is_contiguous()
    assert A.dtype == dtype
    assert x.dtype == dtype
    assert y.dtype == dtype
    assert A.device == x.device == y.device
    assert trans in [CUBLAS_OP_N, CUBLAS_OP_T]
    assert incx > 0 and incy > 0
    assert lda >= n
    if not y.is_cuda:
        raise RuntimeError("flagblas_b200.%s: tensors must live on a CUDA device (there is no CPU path)" % name)

    if m == 0 or n == 0:
        return
    alpha = _scalar(alpha)
    beta = _scalar(beta)
    len_x, len_y = (n, m) if trans == CUBLAS_OP_N else (m, n)
    assert y.numel() >= 1 + (len_y - 1) * incy
    if alpha == 0.0:
        # Only the len_y strided elements are scaled (zero-filled when beta == 0), which is what the
        # reference's tests ask for (tests/test_gemv.py:726-745, 808-836).  Its generic wrapper scales
        # the whole tensor instead (gemv.py:2314-2320); the two differ only for elements that are not
        # part of the vector (between the increments, or past its end).
        _call(code, name, trans, m, n, 0.0, 0, lda, 0, incx, beta, y.data_ptr(), incy, y.device)
        return

    assert x.numel() >= 1 + (len_x - 1) * incx
    assert A.numel() >= (m - 1) * lda + n
    _call(code, name, trans, m, n, alpha, A.data_ptr(), lda, x.data_ptr(), incx, beta, y.data_ptr(), incy, A.device)


def sgemv(trans, m, n, alpha, A, lda, x, incx, beta, y, incy) -> None:
    """fp32 matrix-vector product (reference: ops/level2/gemv.py:2285-2375)."""
    _gemv(_lib.FB_F32, torch.float32, "sgemv", trans, m, n, alpha, A, lda, x, incx, beta, y, incy)


def hgemv(trans, m, n, alpha, A, lda, x, incx, beta, y, incy) -> None:
    """fp16 matrix-vector product, fp32 accumulate, one rounding (reference: ops/level2/gemv.py:2814-2926)."""
    _gemv(_lib.FB_F16, torch.float16, "hgemv", trans, m, n, alpha, A, lda, x, incx, beta, y, incy)


def bfgemv(trans, m, n, alpha, A, lda, x, incx, beta, y, incy) -> None:
    """bf16 matrix-vector product, fp32 accumulate, one rounding (reference: ops/level2/gemv.py:2929-3041)."""
    _gemv(_lib.FB_BF16, torch.bfloat16, "bfgemv", trans, m, n, alpha, A, lda, x, incx, beta, y, incy)


FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
_FP8_CODE = {torch.float8_e4m3fn: _lib.FB_FP8_E4M3, torch.float8_e5m2: _lib.FB_FP8_E5M2}
_Y_CODE = {torch.float32: _lib.FB_F32, torch.float16: _lib.FB_F16, torch.bfloat16: _lib.FB_BF16}


def fp8_gemv(trans, m, n, alpha, A, lda, x, incx, beta, y, incy) -> None:
    """FP8 matrix and vector, ``y[n] = alpha * A.T @ x[m] + beta * y`` with ``y`` in fp32 / fp16 / bf16
    (reference: ops/level2/gemv.py:3044-3124; only ``trans = CUBLAS_OP_T``)."""
    if m == 0 or n == 0:
        return
    assert trans == CUBLAS_OP_T, "FP8 gemv only supports trans=CUBLAS_OP_T (TN format)"
    assert A.stride(1) == 1, "A must be row-major contiguous in the inner dimension"
    assert lda == A.stride(0), "lda must match the row stride of A"
    assert A.dtype in FP8_DTYPES, f"A must be FP8 dtype, got {A.dtype}"
    assert x.dtype in FP8_DTYPES, f"x must be FP8 dtype, got {x.dtype}"
    assert y.dtype in (torch.float32, torch.float16, torch.bfloat16)
    assert A.device == x.device == y.device
    assert m % 16 == 0, f"Matrix dimension m ({m}) must be a multiple of 16 for 16-byte alignment"
    assert n % 16 == 0, f"Matrix dimension n ({n}) must be a multiple of 16 for 16-byte alignment"
    assert lda % 16 == 0, f"lda ({lda}) must be a multiple of 16 for 16-byte alignment"
    assert A.data_ptr() % 16 == 0, "Pointer to A must be 16-byte aligned"
    assert x.data_ptr() % 16 == 0, "Pointer to x must be 16-byte aligned"
    assert y.data_ptr() % 16 == 0, "Pointer to y must be 16-byte aligned"
    assert incx > 0 and incy > 0 and lda >= n
    if not y.is_cuda:
        raise RuntimeError("flagblas_b200.fp8_gemv: tensors must live on a CUDA device (there is no CPU path)")
    alpha = _scalar(alpha)
    beta = _scalar(beta)
    assert y.numel() >= 1 + (n - 1) * incy
    if alpha != 0.0:
        assert x.numel() >= 1 + (m - 1) * incx
    stream, prev = _lib.enter(A.device)
    try:
        ws_bytes = _cop.gemv_fp8_workspace_bytes(m, n) if alpha != 0.0 else 0
        ws_ptr = _lib.scratch(A.device, stream, ws_bytes)
        status = _cop.gemv_fp8(_FP8_CODE[A.dtype], _FP8_CODE[x.dtype], _Y_CODE[y.dtype], m, n, alpha, A.data_ptr(), lda,
                               x.data_ptr(), incx, beta, y.data_ptr(), incy, ws_ptr, ws_bytes, stream)
    finally:
        _lib.leave(prev)
    if status:
        _lib.check(status, "fp8_gemv")
