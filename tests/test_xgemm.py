"""dgemm / cgemm / zgemm: the oracle against vectors the reference's own kernels produced on a B200 (CPU part)
and the CUDA path (operator API -> C ABI) against the oracle and those vectors (GPU part).

Tolerance |got - ref| <= rtol * scale + rtol * |ref| with scale = |alpha| * sqrt(k) * rms(A) * rms(B) + |beta| * rms(C);
rtol 1e-12 for the double-precision types (IEEE FMAs, only the summation order differs) and 1e-5 for complex64
(the reference forms its complex64 products from split-TF32 dots, this library from fp32 FMAs).
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import gpu_cases as gc  # noqa: E402

from oracle import gemm_oracle as go  # noqa: E402

RTOL = {"dgemm": 1e-12, "cgemm": 1e-5, "zgemm": 1e-12}
DEV = "cuda"


@pytest.fixture(scope="module")
def z(golden_dir):
    return np.load(os.path.join(golden_dir, "gpu_reference_xgemm.npz"))


def _rms(t):
    return float(t.abs().pow(2).mean().sqrt()) if t.numel() else 0.0


def _close(got, ref, rtol, scale, what):
    diff = (got - ref).abs()
    bound = rtol * scale + rtol * ref.abs()
    assert bool((diff <= bound).all()), "%s: max diff %g (bound %g)" % (what, float(diff.max()), float(bound.min()))


def _oracle(name, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    c = C.numpy().copy()
    go.gemm_x(gc.XGEMM[name][0], ta, tb, m, n, k, alpha, A.numpy(), lda, B.numpy(), ldb, beta, c, ldc)
    return torch.from_numpy(c)


@pytest.mark.parametrize("name", ["dgemm", "cgemm", "zgemm"])
def test_oracle_vs_reference_on_gpu(z, name):
    for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.xgemm_cases(name):
        np.testing.assert_array_equal(np.concatenate([A.numpy().ravel()[:4], B.numpy().ravel()[:4]]), z[key + "_probe"],
                                      err_msg="input generator differs from the fixture's")
        ref = torch.from_numpy(z[key + "_C"])
        got = _oracle(name, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
        assert torch.equal(ref[:, n:], C[:, n:])                      # the reference leaves the padding alone
        scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B) + abs(beta) * _rms(C)
        # the reference's dgemm / zgemm go through fp64 dots; its cgemm through split-TF32 dots
        _close(got[:, :n], ref[:, :n], 1e-5 if name == "cgemm" else 1e-10, scale, key)


def test_oracle_degenerate_and_conjugate():
    A = np.array([[1 + 2j, 3 - 1j]], dtype=np.complex128)             # 1 x 2
    B = np.array([[2 - 1j], [1j]], dtype=np.complex128)               # 2 x 1
    C = np.zeros((1, 1), dtype=np.complex128)
    go.gemm_x("c128", 0, 0, 1, 1, 2, 1.0, A, 2, B, 1, 0.0, C, 1)
    assert C[0, 0] == (1 + 2j) * (2 - 1j) + (3 - 1j) * 1j
    go.gemm_x("c128", 2, 0, 2, 1, 1, 1.0, A, 2, np.array([[1j]]), 1, 0.0, C2 := np.zeros((2, 1), np.complex128), 1)
    np.testing.assert_array_equal(C2[:, 0], np.conj(A[0]) * 1j)       # op(A) = A^H
    C3 = np.arange(6, dtype=np.float64)
    go.gemm_x("fp64", 0, 0, 0, 3, 2, 1.0, np.zeros(1), 1, np.zeros(1), 1, 0.5, C3, 3)
    np.testing.assert_array_equal(C3, np.arange(6) * 0.5)             # degenerate call scales the whole buffer


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["dgemm", "cgemm", "zgemm"])
def test_against_oracle_and_reference_vectors(z, name):
    import flagblas_b200 as fb
    for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.xgemm_cases(name):
        Cd = C.to(DEV)
        getattr(fb, name)(ta, tb, m, n, k, alpha, A.to(DEV), lda, B.to(DEV), ldb, beta, Cd, ldc)
        torch.cuda.synchronize()
        got = Cd.cpu()
        scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B) + abs(beta) * _rms(C)
        assert torch.equal(got[:, n:], C[:, n:])
        _close(got[:, :n], _oracle(name, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)[:, :n], RTOL[name], scale, key)
        _close(got[:, :n], torch.from_numpy(z[key + "_C"])[:, :n], 1e-5 if name == "cgemm" else 1e-10, scale, key + " vs reference")
    assert fb.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["dgemm", "cgemm", "zgemm"])
def test_shapes_edges_and_early_outs(name):
    import flagblas_b200 as fb
    kind, dt, alpha, beta = gc.XGEMM[name]
    op = getattr(fb, name)
    g = torch.Generator(device="cpu").manual_seed(3)
    ops = (0, 1, 2) if dt.is_complex else (0, 1)
    for (m, n, k) in [(1, 1, 1), (64, 64, 8), (65, 63, 9), (200, 136, 300), (7, 500, 33), (513, 5, 130)]:
        for ta in ops:
            tb = ops[(ta + 1) % len(ops)]
            lda, ldb, ldc = (m if ta else k), (k if tb else n), n
            A = torch.randn((k if ta else m), lda, generator=g, dtype=dt)
            B = torch.randn((n if tb else k), ldb, generator=g, dtype=dt)
            C = torch.randn(m, ldc, generator=g, dtype=dt)
            Cd = C.to(DEV)
            op(ta, tb, m, n, k, alpha, A.to(DEV), lda, B.to(DEV), ldb, beta, Cd, ldc)
            torch.cuda.synchronize()
            scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B) + abs(beta) * _rms(C)
            _close(Cd.cpu(), _oracle(name, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc), RTOL[name], scale,
                   "%s %dx%dx%d t%d%d" % (name, m, n, k, ta, tb))
    # beta == 0 never reads C; alpha == 0 / k == 0 scale the whole buffer; m == 0 too (reference quirk)
    A = torch.ones(4, 4, dtype=dt, device=DEV)
    C = torch.full((4, 4), float("nan"), dtype=dt, device=DEV)
    op(0, 0, 4, 4, 4, 1.0, A, 4, A, 4, 0.0, C, 4)
    assert torch.equal(C.cpu(), torch.full((4, 4), 4.0, dtype=dt))
    op(0, 0, 4, 4, 4, 0.0, A, 4, A, 4, 0.5, C, 4)
    assert torch.equal(C.cpu(), torch.full((4, 4), 2.0, dtype=dt))
    op(0, 0, 2, 2, 0, 1.0, A, 4, A, 4, 2.0, C, 4)
    assert torch.equal(C.cpu(), torch.full((4, 4), 4.0, dtype=dt))
    with pytest.raises(AssertionError):
        op(0, 0, 4, 4, 4, 1.0, A, 3, A, 4, 0.0, C, 4)                 # lda < k
    with pytest.raises(AssertionError):
        op(3, 0, 4, 4, 4, 1.0, A, 4, A, 4, 0.0, C, 4)                 # bad trans
    if not dt.is_complex:
        with pytest.raises(AssertionError):
            op(2, 0, 4, 4, 4, 1.0, A, 4, A, 4, 0.0, C, 4)             # no conjugate transpose for real types
    assert fb.device_status() == 0


# ---------------------------------------------------------------------------------------- trmm
TRMM_RTOL = {"strmm": 1e-5, "dtrmm": 1e-12, "ctrmm": 1e-5, "ztrmm": 1e-12}


def _trmm_oracle(name, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc):
    c = C.numpy().copy()
    go.trmm(gc.TRMM[name][0], side, uplo, trans, diag, m, n, alpha, A.numpy(), lda, B.numpy(), ldb, c, ldc)
    return torch.from_numpy(c)


@pytest.mark.parametrize("name", ["strmm", "dtrmm", "ctrmm", "ztrmm"])
def test_trmm_oracle_vs_reference_on_gpu(z, name):
    for key, (side, uplo, trans, diag, m, n, lda, ldb, ldc, alpha), A, B, C in gc.trmm_cases(name):
        np.testing.assert_array_equal(np.concatenate([A.numpy().ravel()[:4], B.numpy().ravel()[:4]]), z[key + "_probe"])
        ref = torch.from_numpy(z[key + "_C"])
        got = _trmm_oracle(name, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)
        assert torch.equal(ref[:, n:], C[:, n:])
        k = m if side == 0 else n
        scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B)
        _close(got[:, :n], ref[:, :n], 1e-5 if name in ("strmm", "ctrmm") else 1e-10, scale, key)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["strmm", "dtrmm", "ctrmm", "ztrmm"])
def test_trmm_against_oracle_and_reference_vectors(z, name):
    import flagblas_b200 as fb
    for key, (side, uplo, trans, diag, m, n, lda, ldb, ldc, alpha), A, B, C in gc.trmm_cases(name):
        Cd = C.to(DEV)
        getattr(fb, name)(side, uplo, trans, diag, m, n, alpha, A.to(DEV), lda, B.to(DEV), ldb, Cd, ldc)
        torch.cuda.synchronize()
        got = Cd.cpu()
        k = m if side == 0 else n
        scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B)
        assert torch.equal(got[:, n:], C[:, n:])
        _close(got[:, :n], _trmm_oracle(name, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, C, ldc)[:, :n],
               TRMM_RTOL[name], scale, key)
        _close(got[:, :n], torch.from_numpy(z[key + "_C"])[:, :n], 1e-5 if name in ("strmm", "ctrmm") else 1e-10, scale,
               key + " vs reference")
    assert fb.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["strmm", "ztrmm"])
def test_trmm_all_modes_in_place_and_poisoned_triangle(name):
    """Every (side, uplo, trans, diag) combination on ragged sizes; the unused triangle (and, for unit
    diagonals, the diagonal) of A holds NaN and must never be read; B and C may be the same tensor."""
    import flagblas_b200 as fb
    kind, dt, alpha = gc.TRMM[name]
    g = torch.Generator(device="cpu").manual_seed(11)
    for side in (0, 1):
        for uplo in (0, 1):
            for trans in ((0, 1, 2) if dt.is_complex else (0, 1)):
                for diag in (0, 1):
                    m, n = (150, 70) if side == 0 else (70, 150)
                    k = m if side == 0 else n
                    A = torch.randn(k, k, generator=g, dtype=dt)
                    B = torch.randn(m, n, generator=g, dtype=dt)
                    ref = _trmm_oracle(name, side, uplo, trans, diag, m, n, alpha, A, k, B, n, torch.zeros(m, n, dtype=dt), n)
                    Ap = A.clone()
                    mask = torch.tril(torch.ones(k, k), -1).bool() if uplo == 1 else torch.triu(torch.ones(k, k), 1).bool()
                    if diag == 1:
                        mask |= torch.eye(k).bool()
                    Ap[mask] = float("nan")
                    Bd = B.to(DEV)
                    getattr(fb, name)(side, uplo, trans, diag, m, n, alpha, Ap.to(DEV), k, Bd, n, Bd, n)   # in place
                    torch.cuda.synchronize()
                    _close(Bd.cpu(), ref, TRMM_RTOL[name], abs(alpha) * k ** 0.5 * _rms(A) * _rms(B),
                           "%s side=%d uplo=%d trans=%d diag=%d" % (name, side, uplo, trans, diag))
    C = torch.full((8, 8), float("nan"), dtype=dt, device=DEV)
    A = torch.ones(8, 8, dtype=dt, device=DEV)
    getattr(fb, name)(0, 0, 0, 0, 8, 8, 0.0, A, 8, A, 8, C, 8)             # alpha == 0: zero fill
    assert torch.equal(C.cpu(), torch.zeros(8, 8, dtype=dt))
    getattr(fb, name)(0, 0, 0, 0, 0, 8, 1.0, A, 8, A, 8, C, 8)             # m == 0: untouched
    assert torch.equal(C.cpu(), torch.zeros(8, 8, dtype=dt))
    with pytest.raises(AssertionError):
        getattr(fb, name)(2, 0, 0, 0, 8, 8, 1.0, A, 8, A, 8, C, 8)
    assert fb.device_status() == 0


@pytest.mark.gpu
def test_dgemm_tensor_path_and_cuda_core_path_agree(monkeypatch):
    """16-byte aligned fp64 operands take the DMMA kernel; FLAGBLAS_B200_DGEMM_MMA=0 forces the CUDA-core
    kernel.  Both do IEEE FMAs: same tolerance against the oracle, and close agreement with each other."""
    import flagblas_b200 as fb
    g = torch.Generator(device="cpu").manual_seed(17)
    for (m, n, k) in [(128, 64, 16), (130, 66, 50), (512, 384, 1000), (64, 1000, 72), (1000, 30, 256)]:
        for ta in (0, 1):
            for tb in (0, 1):
                lda = ((m if ta else k) + 1) // 2 * 2 + 2
                ldb = ((k if tb else n) + 1) // 2 * 2 + 2
                ldc = n + 1                                           # C may have any pitch
                A = torch.randn((k if ta else m), lda, generator=g, dtype=torch.float64)
                B = torch.randn((n if tb else k), ldb, generator=g, dtype=torch.float64)
                C = torch.randn(m, ldc, generator=g, dtype=torch.float64)
                ref = _oracle("dgemm", ta, tb, m, n, k, 2.5, A, lda, B, ldb, 0.5, C, ldc)
                outs = []
                for mma in ("1", "0"):
                    monkeypatch.setenv("FLAGBLAS_B200_DGEMM_MMA", mma)
                    fb.reload_env()
                    Cd = C.to(DEV)
                    fb.dgemm(ta, tb, m, n, k, 2.5, A.to(DEV), lda, B.to(DEV), ldb, 0.5, Cd, ldc)
                    torch.cuda.synchronize()
                    outs.append(Cd.cpu())
                    scale = 2.5 * k ** 0.5 * _rms(A) * _rms(B) + 0.5 * _rms(C)
                    _close(outs[-1], ref, 1e-12, scale, "dgemm mma=%s %dx%dx%d t%d%d" % (mma, m, n, k, ta, tb))
                assert torch.equal(outs[0][:, n:], C[:, n:])
    assert fb.device_status() == 0


@pytest.mark.gpu
def test_zgemm_tensor_path_and_cuda_core_path_agree(monkeypatch):
    """complex128 on the DMMA kernel (four real MMAs per complex multiply-add) vs the CUDA-core kernel
    (FLAGBLAS_B200_DGEMM_MMA=0): every op combination, ragged sizes, complex alpha and beta."""
    import flagblas_b200 as fb
    g = torch.Generator(device="cpu").manual_seed(19)
    dt = torch.complex128
    alpha, beta = 2.5 + 0.5j, 0.5 - 0.25j
    for (m, n, k) in [(64, 64, 8), (70, 50, 33), (300, 200, 257)]:
        for ta in (0, 1, 2):
            for tb in (0, 1, 2):
                lda, ldb, ldc = (m if ta else k) + 1, (k if tb else n) + 3, n + 1
                A = torch.randn((k if ta else m), lda, generator=g, dtype=dt)
                B = torch.randn((n if tb else k), ldb, generator=g, dtype=dt)
                C = torch.randn(m, ldc, generator=g, dtype=dt)
                ref = _oracle("zgemm", ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
                scale = abs(alpha) * k ** 0.5 * _rms(A) * _rms(B) + abs(beta) * _rms(C)
                for mma in ("1", "0"):
                    monkeypatch.setenv("FLAGBLAS_B200_DGEMM_MMA", mma)
                    fb.reload_env()
                    Cd = C.to(DEV)
                    fb.zgemm(ta, tb, m, n, k, alpha, A.to(DEV), lda, B.to(DEV), ldb, beta, Cd, ldc)
                    torch.cuda.synchronize()
                    _close(Cd.cpu(), ref, 1e-12, scale, "zgemm mma=%s %dx%dx%d t%d%d" % (mma, m, n, k, ta, tb))
    assert fb.device_status() == 0
