"""Randomised shapes for the dense operators: the plan of a call (CTA-pair or 128-row tiles, tile width, cluster
split-K, split through scratch, wide tiles, packed copies of unaligned operands) depends on m, n, k, the leading
dimensions and beta, so a seeded draw over those checks the planner's whole decision space against an fp64 product
of the same (for TF32: truncated) operands.  Padding columns of C must come back untouched."""
import random

import pytest
import torch

import flagblas_b200 as fb
from tests.helpers import KINDS, assert_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"

M_CHOICES = [1, 7, 16, 33, 64, 100, 128, 129, 200, 256, 300, 511, 1024, 1500]
N_CHOICES = [8, 64, 120, 256, 264, 512, 1000, 1536, 2048, 4096, 5000]
K_CHOICES = [64, 128, 192, 520, 1024, 2048, 4096, 6144, 8200, 16384]


# one row block of few rows: A's stage slots shrink to the rows that exist, long k is cut over the CTAs of a cluster,
# which send each other their sums or read them depending on the tile's size
SKINNY_M = [2, 3, 7, 8, 9, 16, 24, 31, 33, 40, 63, 64, 65, 96, 100, 112, 119, 120, 121, 127, 128]
SKINNY_N = [64, 120, 256, 264, 512, 1000, 1536, 2048, 4096, 5000, 6144, 8192]
SKINNY_K = [128, 520, 1024, 2048, 4096, 6144, 8200, 16384]


@pytest.mark.parametrize("chunk", list(range(6)) + ["skinny-0", "skinny-1", "skinny-2"])
def test_random_shapes_match_fp64_product(chunk):
    skinny = isinstance(chunk, str)
    if skinny:
        chunk = 10 + int(chunk[-1])
    rnd = random.Random(1000 + chunk)
    for case in range(25):
        kind = rnd.choice(["bf16", "fp16", "tf32"])
        dt, opname, rtol = KINDS[kind][0], KINDS[kind][1], KINDS[kind][2]
        ta, tb = rnd.randint(0, 1), rnd.randint(0, 1)
        if skinny:
            m, n, k = rnd.choice(SKINNY_M), rnd.choice(SKINNY_N), rnd.choice(SKINNY_K)
        else:
            m, n, k = rnd.choice(M_CHOICES), rnd.choice(N_CHOICES), rnd.choice(K_CHOICES)
        if kind == "tf32":
            k = max(32, k // 2)
        per16 = 16 // (4 if kind == "tf32" else 2)
        pad = rnd.choice([0, 0, per16, 3])                      # 3: pitch not 16-byte aligned -> packed copy
        cols_a, cols_b = (m if ta else k), (k if tb else n)
        lda, ldb, ldc = cols_a + pad, cols_b + pad, n + rnd.choice([0, 0, per16, 1])
        g = torch.Generator(device="cpu").manual_seed(chunk * 100 + case)
        A = (torch.randn((k if ta else m), lda, generator=g) * 0.25).to(dt).to(DEV)
        B = (torch.randn((n if tb else k), ldb, generator=g) * 0.25).to(dt).to(DEV)
        C0 = (torch.randn(m, ldc, generator=g) * 0.5).to(dt).to(DEV)
        alpha, beta = rnd.choice([1.0, 1.5, -0.5]), rnd.choice([0.0, 0.0, 1.0, 0.5])
        C = C0.clone()
        if beta == 0:
            C[:, :n] = float("nan")                              # beta == 0 must not read C
        getattr(fb, opname)(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
        torch.cuda.synchronize()
        what = "%s ta=%d tb=%d %dx%dx%d ld=%d/%d/%d alpha=%g beta=%g" % (kind, ta, tb, m, n, k, lda, ldb, ldc, alpha, beta)
        assert fb.device_status() == 0, what
        op_a = (A[:, :cols_a].t() if ta else A[:, :cols_a]).double()
        op_b = (B[:, :cols_b].t() if tb else B[:, :cols_b]).double()
        if kind == "tf32":
            trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
            op_a, op_b = trunc(op_a), trunc(op_b)
        ref = alpha * (op_a @ op_b)
        if beta != 0:
            ref = ref + beta * C0[:, :n].double()
        scale = abs(alpha) * (k ** 0.5) * 0.25 * 0.25 + abs(beta) * 0.5
        assert_parity(C[:, :n].float().cpu(), ref.float().cpu(), rtol, scale, what)
        assert torch.equal(C[:, n:], C0[:, n:]), what + ": padding columns of C were written"


@pytest.mark.parametrize("chunk", range(2))
def test_random_shapes_sgemm(chunk):
    """The same draw for IEEE fp32 sgemm: 64 x 64 and 128 x 128 tiles, the two-CTA split of k for small problems, the
    register-staged kernel for operands that are not 16-byte aligned."""
    rnd = random.Random(2000 + chunk)
    for case in range(20):
        ta, tb = rnd.randint(0, 1), rnd.randint(0, 1)
        m = rnd.choice([1, 7, 33, 64, 100, 129, 256, 300, 512, 1024])
        n = rnd.choice([8, 64, 120, 256, 264, 512, 1000, 1536])
        k = rnd.choice([16, 100, 256, 260, 512, 1000, 2048, 4100])
        pad = rnd.choice([0, 0, 4, 3])
        cols_a, cols_b = (m if ta else k), (k if tb else n)
        lda, ldb, ldc = cols_a + pad, cols_b + pad, n + rnd.choice([0, 0, 4, 1])
        g = torch.Generator(device="cpu").manual_seed(5000 + chunk * 100 + case)
        A = (torch.randn((k if ta else m), lda, generator=g) * 0.25).to(DEV)
        B = (torch.randn((n if tb else k), ldb, generator=g) * 0.25).to(DEV)
        C0 = (torch.randn(m, ldc, generator=g) * 0.5).to(DEV)
        alpha, beta = rnd.choice([1.0, 1.5, -0.5]), rnd.choice([0.0, 0.0, 1.0, 0.5])
        C = C0.clone()
        if beta == 0:
            C[:, :n] = float("nan")
        fb.sgemm(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
        torch.cuda.synchronize()
        what = "fp32 ta=%d tb=%d %dx%dx%d ld=%d/%d/%d alpha=%g beta=%g" % (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta)
        assert fb.device_status() == 0, what
        op_a = (A[:, :cols_a].t() if ta else A[:, :cols_a]).double()
        op_b = (B[:, :cols_b].t() if tb else B[:, :cols_b]).double()
        ref = alpha * (op_a @ op_b)
        if beta != 0:
            ref = ref + beta * C0[:, :n].double()
        scale = abs(alpha) * (k ** 0.5) * 0.25 * 0.25 + abs(beta) * 0.5
        assert_parity(C[:, :n].cpu(), ref.float().cpu(), KINDS["fp32"][2], scale, what)
        assert torch.equal(C[:, n:], C0[:, n:]), what + ": padding columns of C were written"
