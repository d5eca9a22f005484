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
