"""CPU restatement of the reference's ``sgemv / hgemv / bfgemv``.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module; the product has no CPU path.

Restates ``src/flag_blas/ops/level2/gemv.py``:

* wrapper semantics (``sgemv`` 2285-2375, ``hgemv`` 2814-2926, ``bfgemv`` 2929-3041): ``A`` is a flat
  row-major buffer indexed ``A[i*lda + j]``; ``trans = N`` reads ``x`` at ``j*incx`` and writes ``y`` at
  ``i*incy``; ``trans = T`` swaps the roles; ``m == 0 or n == 0`` returns without touching ``y``;
  ``alpha == 0`` scales the ``len_y`` strided elements of ``y`` by ``beta`` (zero-fill when
  ``beta == 0``) -- the behaviour the reference's tests state (``tests/test_gemv.py:726-745`` and, for
  the elements between the increments on the split-K path, ``808-836``).  The reference's generic
  wrapper applies ``y.zero_()`` / ``y.mul_(beta)`` to the whole tensor (lines 2314-2320, 2329-2333),
  which is the same thing whenever ``y`` holds nothing but the vector (``incy == 1``, exact length);
* kernel arithmetic (``hgemv_n_kernel`` 1475-1531, split-K reduce 1738-1770): fp32 products and sums,
  ``alpha*acc + beta*float(y)`` in fp32 (``alpha*acc`` alone when ``beta == 0``: ``y`` is not read),
  one rounding to the storage type.

The sum is formed in float64 and narrowed to float32 before the epilogue; the reference adds fp32
chunks in an order that depends on its tuned block sizes, so the two differ by a few fp32 ulps of the
partial sums.  Pinned by the vectors in ``tests/golden/gpu_reference_gemv.npz``, which
the reference's own kernels produced on a B200 (``tests/golden/make_golden_gpu.py gemv``).
"""
import numpy as np

from .gemm_oracle import _ROUND_OUT, OP_N, OP_T

_KIND = {"sgemv": "fp32", "hgemv": "fp16", "bfgemv": "bf16"}


def gemv(name, trans, m, n, alpha, A, lda, x, incx, beta, y, incy, out_kind=None):
    """In place on the flat numpy buffer ``y``; returns None like the reference.

    ``name = "fp8_gemv"`` (``gemv.py:3044-3124``; kernel 2158-2220): ``A`` and ``x`` hold decoded FP8
    values, ``trans`` must be T, ``out_kind`` ("fp32" / "fp16" / "bf16") is the storage type of ``y``;
    the arithmetic is the same fp32 accumulate and single rounding."""
    kind = out_kind if name == "fp8_gemv" else _KIND[name]
    assert name != "fp8_gemv" or trans == OP_T
    assert trans in (OP_N, OP_T) and incx > 0 and incy > 0 and lda >= n
    if m == 0 or n == 0:
        return None
    alpha = float(alpha)
    beta = float(beta)
    yf = y.reshape(-1)
    len_x, len_y = (n, m) if trans == OP_N else (m, n)
    ys = yf[: 1 + (len_y - 1) * incy : incy]
    if alpha == 0.0:
        if beta == 0.0:
            ys[...] = 0
        elif beta != 1.0:
            ys[...] = _ROUND_OUT[kind](np.float32(beta) * ys.astype(np.float32))
        return None
    af = A.reshape(-1)
    need = (m - 1) * lda + n
    a = np.zeros((m, lda), dtype=np.float64).reshape(-1)
    a[:need] = af[:need]
    a = a.reshape(m, lda)[:, :n]
    xv = x.reshape(-1)[: 1 + (len_x - 1) * incx : incx].astype(np.float64)
    acc = (a @ xv if trans == OP_N else a.T @ xv).astype(np.float32)
    res = np.float32(alpha) * acc
    if beta != 0.0:
        res = res + np.float32(beta) * ys.astype(np.float32)
    ys[...] = _ROUND_OUT[kind](res)
    return None


def gemv_fp64(trans, m, n, alpha, A, lda, x, incx, beta, y, incy):
    """Accuracy yard-stick: the same product entirely in float64, no rounding; returns the len_y vector."""
    af = A.reshape(-1).astype(np.float64)
    a = np.zeros(m * lda)
    a[: (m - 1) * lda + n] = af[: (m - 1) * lda + n]
    a = a.reshape(m, lda)[:, :n]
    len_x, len_y = (n, m) if trans == OP_N else (m, n)
    xv = x.reshape(-1)[: 1 + (len_x - 1) * incx : incx].astype(np.float64)
    ys = y.reshape(-1)[: 1 + (len_y - 1) * incy : incy].astype(np.float64)
    return float(alpha) * (a @ xv if trans == OP_N else a.T @ xv) + float(beta) * ys
