"""CPU restatement of the reference's GEMM-family semantics.  TEST INFRASTRUCTURE ONLY.

This module is the checker the parity tests, the smoke test and the CPU-baseline
leg of the benchmark compare against.  Nothing in the product package imports it;
the product has no CPU path.

It restates, in numpy, what the reference's operators compute:

* dense ``sgemm / hgemm / bfgemm`` -- wrapper semantics of
  ``src/flag_blas/ops/level3/hgemm.py:473-529`` (early-outs that scale the whole
  ``C`` buffer, ``C`` never read when ``beta == 0``) and kernel arithmetic of
  ``hgemm.py:44-143`` (fp32 accumulator, ``alpha*acc + beta*float(c)`` in fp32,
  one rounding to the storage type);
* ``group_bfgemm / group_hgemm`` -- ``src/flag_blas/ops/level3/group_gemm.py:131-218``
  (per-group pointers and strides, ``ori_c*beta + acc*alpha``, C skipped when
  ``beta == 0``); ``group_tf32gemm`` -- ``group_gemm.py:427-537`` (``B_g`` stored
  ``[n_g, k_g]``, inputs rounded to TF32 before the product);
* ``group_mm`` -- ``group_gemm.py:587-717`` (cumulative int32 row offsets).

Values travel as numpy float32/float64 arrays that are exactly representable in
the storage type being modelled ("fp32", "tf32", "fp16", "bf16"); outputs are
rounded once to that type.  The accumulator is formed in float64 and narrowed
to float32 before the epilogue, which differs from the reference's fp32
chunk-wise accumulation by a few fp32 ulps of the partial sums -- far inside
every tolerance used and pinned by the golden vectors in ``tests/golden``: fp32 / fp16 vectors made
by the reference's own kernels under Triton's CPU interpreter (``make_golden.py``), and bf16 / fp16 /
fp32 / TF32 vectors made by the same kernels running natively on a B200 (``make_golden_gpu.py``).
The latter show that on B200 the reference's TF32 dots TRUNCATE their fp32 operands (the operands go
from shared memory straight into the tensor core), hence ``tf32_mode="trunc"`` is the default here;
``"rna"`` (round to nearest, what a register-operand lowering does) and ``"none"`` are kept for
comparison.
"""
import numpy as np

OP_N, OP_T = 0, 1


# ------------------------------------------------------------------ rounding
def round_bf16(x):
    """Round-to-nearest-even to bfloat16, returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    bias = np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    r = ((u + bias) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isnan(x), x, r).astype(np.float32)


def round_fp16(x):
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_tf32(x):
    """fp32 -> tf32 the way ``cvt.rna.tf32.f32`` does (nearest, ties away from zero)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    r = ((u + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)
    return np.where(np.isfinite(x), r, x).astype(np.float32)


def trunc_tf32(x):
    """fp32 -> tf32 by dropping the 13 low mantissa bits (what a tensor core does to raw fp32 words)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


_ROUND_OUT = {
    "fp32": lambda x: np.asarray(x, dtype=np.float32),
    "tf32": lambda x: np.asarray(x, dtype=np.float32),
    "fp16": round_fp16,
    "bf16": round_bf16,
}


def _epilogue(acc64, alpha, beta, c, kind):
    """(alpha*acc + beta*float(C)) in fp32, one rounding (hgemm.py:128-143)."""
    acc = acc64.astype(np.float32)
    res = np.float32(alpha) * acc
    if beta != 0.0:
        res = res + np.float32(beta) * c.astype(np.float32)
    return _ROUND_OUT[kind](res)


def _inputs(a, kind, tf32_mode):
    if kind == "tf32":
        a = round_tf32(a) if tf32_mode == "rna" else (trunc_tf32(a) if tf32_mode == "trunc" else a)
    return np.asarray(a, dtype=np.float64)


# --------------------------------------------------------------------- dense
def gemm(kind, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, tf32_mode="trunc"):
    """In-place dense GEMM on flat row-major buffers; returns None like the reference.

    ``A``, ``B``, ``C`` are 1-D (or any-shape, C-contiguous) numpy arrays that are
    reinterpreted as flat buffers, exactly as the reference's kernels index raw
    pointers with ``lda/ldb/ldc``.
    """
    assert transa in (OP_N, OP_T) and transb in (OP_N, OP_T)
    alpha = float(alpha)
    beta = float(beta)
    cf = C.reshape(-1)
    # early-outs scale the WHOLE C buffer (sgemm.py:449-454)
    if m == 0 or n == 0 or k == 0 or alpha == 0.0:
        if beta == 0.0:
            cf[...] = 0
        elif beta != 1.0:
            cf[...] = _ROUND_OUT[kind](np.float32(beta) * cf.astype(np.float32))
        return None
    af = A.reshape(-1)
    bf = B.reshape(-1)
    if transa == OP_N:
        a = af[: m * lda].reshape(m, lda)[:, :k]
    else:
        a = af[: k * lda].reshape(k, lda)[:, :m].T
    if transb == OP_N:
        b = bf[: k * ldb].reshape(k, ldb)[:, :n]
    else:
        b = bf[: n * ldb].reshape(n, ldb)[:, :k].T
    acc = _inputs(a, kind, tf32_mode) @ _inputs(b, kind, tf32_mode)
    cv = cf[: m * ldc].reshape(m, ldc)[:, :n]
    cv[...] = _epilogue(acc, alpha, beta, cv, kind)
    return None


def gemm_fp64(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    """Accuracy yard-stick: the same contraction entirely in float64, no rounding; returns [m, n]."""
    af, bf, cf = A.reshape(-1), B.reshape(-1), C.reshape(-1)
    a = af[: m * lda].reshape(m, lda)[:, :k] if transa == OP_N else af[: k * lda].reshape(k, lda)[:, :m].T
    b = bf[: k * ldb].reshape(k, ldb)[:, :n] if transb == OP_N else bf[: n * ldb].reshape(n, ldb)[:, :k].T
    res = float(alpha) * (a.astype(np.float64) @ b.astype(np.float64))
    if beta != 0.0:
        res = res + float(beta) * cf[: m * ldc].reshape(m, ldc)[:, :n].astype(np.float64)
    return res


# ------------------------------------------------------------------- grouped
def group_gemm(kind, a_list, b_list, c_list, alpha, beta, b_stored_nk=False, tf32_mode="trunc"):
    """Per-group ``out_g = alpha * A_g @ B_g + beta * C_g`` (group_gemm.py:131-218, 488-504).

    ``a_list[g]`` is ``[m_g, k_g]``; ``b_list[g]`` is ``[k_g, n_g]``, or ``[n_g, k_g]`` when
    ``b_stored_nk`` (the group_tf32gemm layout); ``c_list[g]`` is ``[m_g, n_g]`` and is not
    read when ``beta == 0``.  Returns the list of outputs.
    """
    outs = []
    for a, b, c in zip(a_list, b_list, c_list):
        bm = b.T if b_stored_nk else b
        m, n = a.shape[0], bm.shape[1]
        if m == 0 or n == 0:
            outs.append(np.zeros((m, n), dtype=np.float32))
            continue
        acc = _inputs(a, kind, tf32_mode) @ _inputs(bm, kind, tf32_mode)
        outs.append(_epilogue(acc, float(alpha), float(beta), c if beta != 0.0 else None, kind))
    return outs


def group_mm(kind, A, B, offs, tf32_mode="trunc"):
    """``C[o_{g-1}:o_g] = A[o_{g-1}:o_g] @ B[g]`` (group_gemm.py:614-686); rows past offs[-1] stay 0.
    The reference's kernel forms the products in the storage precision (``tl.dot(..., allow_tf32=False)``,
    ``group_gemm.py:656``): kinds "fp16" / "bf16" / "fp32" model that.  ``kind == "tf32"`` models what the CUDA
    library does with fp32 tensors -- TF32 tensor-core products, operands truncated as in ``group_tf32gemm`` --
    an extension the reference does not have."""
    M, N = A.shape[0], B.shape[2]
    C = np.zeros((M, N), dtype=np.float32)
    start = 0
    for g, end in enumerate(int(e) for e in offs):
        if end > start:
            acc = _inputs(A[start:end], kind, tf32_mode) @ _inputs(B[g], kind, tf32_mode)
            C[start:end] = _epilogue(acc, 1.0, 0.0, None, kind)
        start = end
    return C


# ------------------------------------------------------- double / complex dense GEMM
_X_DTYPE = {"fp64": np.float64, "c64": np.complex64, "c128": np.complex128}


def gemm_x(kind, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    """``dgemm`` / ``cgemm`` / ``zgemm`` (``ops/level3/dgemm.py:160-208``, ``cgemm.py:192-254``,
    ``zgemm.py:192-254``) on flat row-major numpy buffers of dtype float64 / complex64 / complex128,
    in place on ``C``.  ``trans`` 0 = N, 1 = T, 2 = C (conjugate transpose, complex kinds only).  The same
    early-outs as the other dense operators: a degenerate call scales the whole ``C`` buffer.  The
    contraction is formed in float64 / complex128 and rounded once to the storage type."""
    dt = _X_DTYPE[kind]
    cplx = kind != "fp64"
    assert transa in ((0, 1, 2) if cplx else (0, 1)) and transb in ((0, 1, 2) if cplx else (0, 1))
    alpha = complex(alpha) if cplx else float(alpha)
    beta = complex(beta) if cplx else float(beta)
    cf = C.reshape(-1)
    if m == 0 or n == 0 or k == 0 or alpha == 0:
        if beta == 0:
            cf[...] = 0
        elif beta != 1:
            cf[...] = (beta * cf.astype(np.complex128 if cplx else np.float64)).astype(dt)
        return None
    wide = np.complex128 if cplx else np.float64
    af, bf = A.reshape(-1).astype(wide), B.reshape(-1).astype(wide)

    def view(buf, rows, cols, ld):
        full = np.zeros(rows * ld, dtype=wide)
        need = (rows - 1) * ld + cols
        full[:need] = buf[:need]
        return full.reshape(rows, ld)[:, :cols]

    a = view(af, m, k, lda) if transa == 0 else view(af, k, m, lda).T
    b = view(bf, k, n, ldb) if transb == 0 else view(bf, n, k, ldb).T
    if transa == 2:
        a = a.conj()
    if transb == 2:
        b = b.conj()
    acc = a @ b
    need_c = (m - 1) * ldc + n
    cfull = np.zeros(m * ldc, dtype=wide)
    cfull[:need_c] = cf[:need_c]
    cv = cfull.reshape(m, ldc)[:, :n]
    res = alpha * acc + (beta * cv if beta != 0 else 0)
    out = np.zeros(m * ldc, dtype=dt)
    out[:need_c] = cf[:need_c]
    out2 = out.reshape(m, ldc)
    out2[:, :n] = res.astype(dt)
    cf[:need_c] = out[:need_c]
    return None


_T_DTYPE = {"fp32": np.float32, "fp64": np.float64, "c64": np.complex64, "c128": np.complex128}


def trmm(kind, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc):
    """``strmm`` / ``dtrmm`` / ``ctrmm`` / ``ztrmm`` (``ops/level3/trmm.py:39-196`` generic kernel, wrappers
    ``:2095-2231`` ...): ``C[:m, :n] = alpha * op(tri(A)) @ B`` (``side`` 0) or ``alpha * B @ op(tri(A))``
    (``side`` 1) on flat row-major numpy buffers, in place on ``C``; ``uplo`` 0 = lower, 1 = upper triangle of
    the stored ``A``; ``diag`` 1 = unit diagonal; ``trans`` 0 / 1 / 2 = N / T / C.  ``m == 0 or n == 0``
    leaves ``C`` alone, ``alpha == 0`` zero-fills the block.  Formed in float64 / complex128, rounded once."""
    dt = _T_DTYPE[kind]
    if m == 0 or n == 0:
        return None
    wide = np.complex128 if kind in ("c64", "c128") else np.float64
    kdim = m if side == 0 else n
    cf = C.reshape(-1)
    cv = cf[: m * ldc].reshape(m, ldc)[:, :n]
    if alpha == 0:
        cv[...] = 0
        return None
    a = A.reshape(-1)[: kdim * lda].reshape(kdim, lda)[:, :kdim].astype(wide)
    a = np.triu(a) if uplo == 1 else np.tril(a)
    if diag == 1:
        a = a - np.diag(np.diag(a)) + np.eye(kdim, dtype=wide)
    if trans == 1:
        a = a.T
    elif trans == 2:
        a = a.conj().T
    b = B.reshape(-1)[: m * ldb].reshape(m, ldb)[:, :n].astype(wide)
    res = alpha * (a @ b if side == 0 else b @ a)
    cv[...] = res.astype(dt)
    return None
