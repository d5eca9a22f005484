"""The large and the unaligned entries of the reference's own shape lists, at size.

Dense: ``tests/accuracy_utils.py:332-357`` of the reference (4095^3, 8191^3, (4097, 8191, 4095), the LLM shapes
(8192, 28672, 8192) and (4096, 8192, 28672), the skinny (32768, 1024, 1024)) with its alpha / beta pairs
(``tests/test_sgemm.py:218-220``: 2.5 / 0.5 for fp32, 1.5 / 0.5 for the 16-bit types), NN and NT, all four arithmetic
types.  Grouped: three of its ``(k, e, n)`` configurations with e = 128 and 512 groups and ``m_g`` up to 4096
(``tests/accuracy_utils.py:299-330``; the reference draws ``m_g`` unseeded, here the draw is seeded).
Checked through whole rows and columns against fp64, so the suite stays within minutes.
"""
import random

import pytest
import torch

import flagblas_b200 as fb
from tests.helpers import KINDS, assert_parity, check_samples_fp64

pytestmark = pytest.mark.gpu
DEV = "cuda"

DENSE_SHAPES = [(4095, 4095, 4095), (8191, 8191, 8191), (4097, 8191, 4095), (8192, 28672, 8192), (4096, 8192, 28672),
                (32768, 1024, 1024)]


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("shape", DENSE_SHAPES, ids=lambda s: "x".join(str(v) for v in s))
def test_reference_dense_shapes_at_size(kind, shape):
    m, n, k = shape
    dt, opname, _ = KINDS[kind]
    alpha, beta = (2.5, 0.5) if kind == "fp32" else (1.5, 0.5)
    op = getattr(fb, opname)
    g = torch.Generator(device=DEV).manual_seed(m + 3 * n + 7 * k)
    for ta, tb in ((0, 0), (0, 1)):
        A = (torch.randn((k, m) if ta else (m, k), generator=g, device=DEV) * 0.5).to(dt)
        B = (torch.randn((n, k) if tb else (k, n), generator=g, device=DEV) * 0.5).to(dt)
        C0 = torch.randn(m, n, generator=g, device=DEV).to(dt)
        C = C0.clone()
        op(ta, tb, m, n, k, alpha, A, A.shape[1], B, B.shape[1], beta, C, n)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        scale = abs(alpha) * k ** 0.5 * 0.25 + abs(beta)
        if kind == "fp32":
            # the yard-stick is an fp64 product; an fp32 accumulator (the reference's too) drifts from it by about
            # sqrt(k) roundings of the running sum, which passes 1e-5 of the typical output size beyond k ~ 8192
            scale *= max(1.0, k / 8192.0)
        check_samples_fp64(kind, ta, tb, m, n, k, alpha, beta, A, B, C0, C, scale, "%s %dx%dx%d t%d%d" % (kind, m, n, k, ta, tb))
        del A, B, C0, C


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
@pytest.mark.parametrize("cfg", [(1024, 128, 2048), (2048, 512, 512), (7168, 128, 256)], ids=lambda c: "k%d_e%d_n%d" % c)
def test_reference_grouped_shapes_at_size(kind, cfg):
    K, E, N = cfg
    dt = KINDS[kind][0]
    nk = kind == "tf32"                      # group_tf32gemm stores B_g as [n, k]
    rnd = random.Random(50)
    ms = [rnd.randint(1, 4096) for _ in range(E)]
    T = sum(ms)
    g = torch.Generator(device=DEV).manual_seed(K + E + N)
    A = torch.randn(T, K, generator=g, device=DEV).to(dt)
    B = (torch.randn(E, N, K, generator=g, device=DEV) if nk else torch.randn(E, K, N, generator=g, device=DEV))
    B = (B * K ** -0.5).to(dt)
    C = torch.randn(T, N, generator=g, device=DEV).to(dt)
    out = torch.full_like(C, float("nan"))
    es = A.element_size()
    starts = [sum(ms[:e]) for e in range(E)]
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=DEV)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    fn = getattr(fb, {"bf16": "group_bfgemm", "fp16": "group_hgemm", "tf32": "group_tf32gemm"}[kind])
    fn(out, i64([A.data_ptr() + s * K * es for s in starts]), i64([B.data_ptr() + e * K * N * es for e in range(E)]),
       i64([C.data_ptr() + s * N * es for s in starts]), i64([out.data_ptr() + s * N * es for s in starts]), i32(ms),
       i32([N] * E), i32([K] * E), i32([K] * E), i32([K if nk else N] * E), i32([N] * E), E, T, N, K, 1.5, 0.5)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert not torch.isnan(out).any()
    trunc = (lambda x: (x.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)) if kind == "tf32" else (lambda x: x)
    for e in range(E):
        s, mg = starts[e], ms[e]
        rows = sorted({s, s + mg // 2, s + mg - 1, s + min(mg - 1, 255), s + (mg - 1) // 256 * 256})
        Be = trunc(B[e]).double()
        ref = 1.5 * (trunc(A[rows]).double() @ (Be.t() if nk else Be)) + 0.5 * C[rows].double()
        assert_parity(out[rows].float().cpu(), ref.float().cpu(), KINDS[kind][2], 2.0, "%s group %d of %s" % (kind, e, cfg))
