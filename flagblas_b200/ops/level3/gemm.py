"""Dense GEMM operators: ``sgemm``, ``hgemm``, ``bfgemm``, ``tf32gemm``.

Same call signature and semantics as the reference operators
(``src/flag_blas/ops/level3/sgemm.py:421-477``, ``hgemm.py:473-529``,
``bfgemm.py:473-529`` and their Hopper overrides
``src/flag_blas/runtime/backend/_nvidia/hopper/ops/{sgemm,hgemm,bfgemm}.py``):

    X(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None

row-major matrices, ``ld*`` = row stride in elements, in place on ``C``.
``tf32gemm`` is the dense form of what the reference only offers grouped
(``group_tf32gemm``, ``ops/level3/group_gemm.py:427-581``): fp32 storage, TF32
tensor-core products, fp32 accumulation.

The arithmetic runs in the native library through its C ABI (``fb_gemm``, reached via the
pybind11 module ``c_operators``); this module only validates arguments the way the reference does and hands over raw
addresses and the current CUDA stream.
"""
import torch

from ... import _lib
from .._constants import CUBLAS_OP_N, CUBLAS_OP_T

_cop = _lib.cop


def _scalar(x):
    # A 0-dim tensor costs a host sync here, exactly as in the reference (hgemm.py:498-499).
    return x.item() if isinstance(x, torch.Tensor) else float(x)


def _scale_whole(C, beta, code):
    """Reference quirk (sgemm.py:449-454): a degenerate call scales *every* element of C."""
    if beta == 1.0 or C.numel() == 0:
        return
    numel = C.numel()
    # k == 0 makes fb_gemm scale the (1 x numel) block by beta (zero-fill when beta == 0).
    _launch(code, "scale", 0, 0, 1, numel, 0, 0.0, 0, 1, 0, numel, beta, C.data_ptr(), numel, C.device)


def _validate(dtype, name, transa, transb, m, n, k, A, lda, B, ldb, C, ldc):
    """Argument checks of the reference wrappers (AssertionError on violation)."""
    assert A.is_contiguous()
    assert B.is_contiguous()
    assert C.is_contiguous()
    assert A.dtype == dtype
    assert B.dtype == dtype
    assert C.dtype == dtype
    assert A.device == B.device == C.device
    assert transa in [CUBLAS_OP_N, CUBLAS_OP_T]
    assert transb in [CUBLAS_OP_N, CUBLAS_OP_T]
    if not C.is_cuda:
        raise RuntimeError("flagblas_b200.%s: tensors must live on a CUDA device (there is no CPU path)" % name)


def _validate_extents(transa, transb, m, n, k, A, lda, B, ldb, C, ldc):
    """Leading-dimension / buffer-size checks of the reference's Hopper wrappers
    (runtime/backend/_nvidia/hopper/ops/sgemm.py:1554-1569)."""
    if transa == CUBLAS_OP_N:
        assert lda >= k
        assert A.numel() >= m * lda
    else:
        assert lda >= m
        assert A.numel() >= k * lda
    if transb == CUBLAS_OP_N:
        assert ldb >= n
        assert B.numel() >= k * ldb
    else:
        assert ldb >= k
        assert B.numel() >= n * ldb
    assert ldc >= n
    assert C.numel() >= m * ldc


def _launch(code, name, transa, transb, m, n, k, alpha, a_ptr, lda, b_ptr, ldb, beta, c_ptr, ldc, device):
    """Enqueue one fb_gemm on the current stream of ``device`` from raw addresses."""
    stream, prev = _lib.enter(device)
    try:
        # packed copies of operands TMA cannot address in place, if any, go to per-stream scratch
        ws_bytes = _cop.gemm_workspace_bytes(code, transa, transb, m, n, k, a_ptr, lda, b_ptr, ldb)
        ws_ptr = _lib.scratch(device, stream, ws_bytes)
        status = _cop.gemm(code, transa, transb, m, n, k, alpha, a_ptr, lda, b_ptr, ldb, beta, c_ptr, ldc, ws_ptr,
                           ws_bytes, stream)
    finally:
        _lib.leave(prev)
    if status:
        _lib.check(status, name)


def _gemm(code, dtype, name, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    _validate(dtype, name, transa, transb, m, n, k, A, lda, B, ldb, C, ldc)
    alpha = _scalar(alpha)
    beta = _scalar(beta)
    if m == 0 or n == 0 or k == 0 or alpha == 0.0:
        _scale_whole(C, beta, code)
        return
    _validate_extents(transa, transb, m, n, k, A, lda, B, ldb, C, ldc)
    _launch(code, name, transa, transb, m, n, k, alpha, A.data_ptr(), lda, B.data_ptr(), ldb, beta, C.data_ptr(),
            ldc, A.device)


OPS = {
    "sgemm": (_lib.FB_F32, torch.float32),
    "tf32gemm": (_lib.FB_TF32, torch.float32),
    "hgemm": (_lib.FB_F16, torch.float16),
    "bfgemm": (_lib.FB_BF16, torch.bfloat16),
}


def sgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """fp32 GEMM with IEEE single-precision products (reference: ops/level3/sgemm.py:421-477)."""
    _gemm(_lib.FB_F32, torch.float32, "sgemm", transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)


def tf32gemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """fp32-storage GEMM with TF32 tensor-core products and fp32 accumulation."""
    _gemm(_lib.FB_TF32, torch.float32, "tf32gemm", transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)


def hgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """fp16 GEMM, fp32 accumulate, one rounding (reference: ops/level3/hgemm.py:473-529)."""
    _gemm(_lib.FB_F16, torch.float16, "hgemm", transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)


def bfgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc) -> None:
    """bf16 GEMM, fp32 accumulate, one rounding (reference: ops/level3/bfgemm.py:473-529)."""
    _gemm(_lib.FB_BF16, torch.bfloat16, "bfgemm", transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
