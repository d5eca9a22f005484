"""Shared helpers of the parity tests: seeded inputs, the tolerance rule, oracle glue."""
import numpy as np
import torch

from oracle import gemm_oracle as go

KINDS = {
    # kind: (torch dtype, operator name, rtol against the oracle)
    "fp32": (torch.float32, "sgemm", 1e-5),
    "tf32": (torch.float32, "tf32gemm", 1e-3),
    "fp16": (torch.float16, "hgemm", 1e-2),
    "bf16": (torch.bfloat16, "bfgemm", 1e-2),
}


def make_dense(kind, ta, tb, m, n, k, pad=0, seed=0, scale=1.0, c_nan=False):
    """Seeded row-major operands (CPU tensors) with leading dimensions padded by ``pad``."""
    dt = KINDS[kind][0]
    g = torch.Generator(device="cpu").manual_seed(seed)
    lda = (m if ta else k) + pad
    ldb = (k if tb else n) + pad
    ldc = n + pad
    A = (torch.randn((k if ta else m), lda, generator=g) * scale).to(dt)
    B = (torch.randn((n if tb else k), ldb, generator=g) * scale).to(dt)
    C = torch.randn(m, ldc, generator=g).to(dt)
    if c_nan:
        C.fill_(float("nan"))
    return A, lda, B, ldb, C, ldc


def oracle_dense(kind, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, tf32_mode="trunc"):
    """Run the oracle on copies of CPU tensors; returns the resulting C as a float32 tensor."""
    a, b, c = A.float().numpy().copy(), B.float().numpy().copy(), C.float().numpy().copy()
    go.gemm(kind, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, tf32_mode=tf32_mode)
    return torch.from_numpy(c)


def result_scale(k, A, B, alpha):
    """Typical magnitude of one output element: |alpha| * sqrt(k) * rms(A) * rms(B)."""
    ra = float(A.float().pow(2).mean().sqrt()) if A.numel() else 0.0
    rb = float(B.float().pow(2).mean().sqrt()) if B.numel() else 0.0
    return abs(alpha) * (max(k, 1) ** 0.5) * ra * rb


def assert_parity(got, ref, rtol, scale, what=""):
    """|got - ref| <= rtol * scale + rtol * |ref|, elementwise, NaNs must coincide.

    ``scale`` is the typical output magnitude (see result_scale): entries of a GEMM
    with zero-mean inputs can be arbitrarily close to zero, so a purely relative bound
    is meaningless there; the absolute term is the same rtol applied to the typical size.
    """
    got = got.double()
    ref = ref.double()
    assert got.shape == ref.shape, what
    nan_g, nan_r = torch.isnan(got), torch.isnan(ref)
    assert torch.equal(nan_g, nan_r), "%s: NaN pattern differs" % what
    diff = (got - ref).abs()
    bound = rtol * scale + rtol * ref.abs()
    bad = (diff > bound) & ~nan_r
    if bad.any():
        i = int(torch.nonzero(bad.reshape(-1))[0])
        raise AssertionError("%s: %d / %d elements out of tolerance; first at flat %d: got %r ref %r (bound %g); "
                             "max diff %g" % (what, int(bad.sum()), bad.numel(), i, float(got.reshape(-1)[i]),
                                              float(ref.reshape(-1)[i]), float(bound.reshape(-1)[i]),
                                              float(diff[~nan_r].max())))


def check_samples_fp64(kind, ta, tb, m, n, k, alpha, beta, A, B, C0, C, scale, what, dev="cuda"):
    """Whole rows and whole columns of a device-resident result ``C`` against an fp64 product of the same operands
    (TF32: with the 13 low mantissa bits of the operands dropped, as the tensor core does), formed on the GPU block
    by block so that sizes the numpy oracle cannot finish stay cheap.  ``A``, ``B`` in storage layout, ``C0`` = C
    before the call (ignored when ``beta == 0``)."""
    rtol = KINDS[kind][2]
    rows = torch.tensor(sorted(r for r in {0, 1, 127, 128, 255, 256, m // 2 + 3, m - 2, m - 1} if 0 <= r < m), device=dev)
    cols = torch.tensor(sorted(c for c in {0, 1, 255, 256, 511, 512, n // 2 + 5, n - 2, n - 1} if 0 <= c < n), device=dev)
    trunc = (lambda x: (x.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)) if kind == "tf32" else (lambda x: x)
    a_rows = trunc(A[:, rows].t() if ta else A[rows]).double()            # [rows, k]
    b_cols = trunc(B[cols].t() if tb else B[:, cols]).double()            # [k, cols]
    ref_rows = torch.empty(len(rows), n, dtype=torch.float64, device=dev)
    ref_cols = torch.empty(m, len(cols), dtype=torch.float64, device=dev)
    step = 2048
    for j in range(0, n, step):
        bj = trunc(B[j:j + step].t() if tb else B[:, j:j + step]).double()
        ref_rows[:, j:j + step] = alpha * (a_rows @ bj)
    for i in range(0, m, step):
        ai = trunc(A[:, i:i + step].t() if ta else A[i:i + step]).double()
        ref_cols[i:i + step] = alpha * (ai @ b_cols)
    if beta != 0.0:
        ref_rows += beta * C0[rows, :n].double()
        ref_cols += beta * C0[:, cols].double()
    assert_parity(C[rows, :n].float().cpu(), ref_rows.float().cpu(), rtol, scale, what + " rows")
    assert_parity(C[:, cols].float().cpu(), ref_cols.float().cpu(), rtol, scale, what + " cols")
