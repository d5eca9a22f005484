"""sgemv / hgemv / bfgemv: the oracle against the vectors the reference's own kernels produced on a
B200 (CPU part), and the CUDA path (operator API -> C ABI) against the oracle, against those vectors
and through size-independent properties (GPU part).

Tolerances: |got - ref| <= rtol * scale + rtol * |ref| with scale = |alpha| * sqrt(len_x) * rms(A) * rms(x)
(+ |beta| * rms(y)); rtol 1e-5 for sgemv, 1e-2 for hgemv / bfgemv (one rounding of an fp32 result:
the typical difference is one unit in the last place of the 16-bit type).
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import gpu_cases as gc  # noqa: E402

from oracle import gemv_oracle as gvo  # noqa: E402
from tests.helpers import assert_parity  # noqa: E402

NAMES = {"sgemv": (torch.float32, 1e-5), "hgemv": (torch.float16, 1e-2), "bfgemv": (torch.bfloat16, 1e-2)}
DEV = "cuda"


@pytest.fixture(scope="module")
def z(golden_dir):
    return np.load(os.path.join(golden_dir, "gpu_reference_gemv.npz"))


def _scale(len_x, A, x, y, alpha, beta):
    rms = lambda t: float(t.float().pow(2).mean().sqrt()) if t.numel() else 0.0  # noqa: E731
    return abs(alpha) * (len_x ** 0.5) * rms(A) * rms(x) + abs(beta) * rms(y)


def _oracle(name, trans, m, n, alpha, A, lda, x, incx, beta, y, incy):
    yy = y.float().numpy().copy()
    gvo.gemv(name, trans, m, n, alpha, A.float().numpy(), lda, x.float().numpy(), incx, beta, yy, incy)
    return torch.from_numpy(yy)


def _make(name, trans, m, n, pad, incx, incy, seed, extra_y=0, y_nan=False):
    dt = NAMES[name][0]
    g = torch.Generator(device="cpu").manual_seed(seed)
    lda = n + pad
    len_x, len_y = (n, m) if trans == 0 else (m, n)
    A = torch.randn(max(m, 1), max(lda, 1), generator=g).to(dt)
    x = torch.randn(1 + (max(len_x, 1) - 1) * incx, generator=g).to(dt)
    y = torch.randn(1 + (max(len_y, 1) - 1) * incy + extra_y, generator=g).to(dt)
    if y_nan:
        y[: 1 + (max(len_y, 1) - 1) * incy : incy] = float("nan")
    return A, lda, x, y


# --------------------------------------------------------------------------------- oracle (CPU)
@pytest.mark.parametrize("name", list(NAMES))
def test_oracle_vs_reference_on_gpu(z, name):
    for key, (trans, m, n, lda, incx, incy, alpha, beta), A, x, y in gc.gemv_cases(name):
        probe = np.concatenate([A.float().numpy().ravel()[:8], x.float().numpy().ravel()[:1]])
        np.testing.assert_array_equal(probe, z[key + "_probe"], err_msg="input generator differs from the fixture's")
        ref = gc.unpack(z[key + "_y"], gc.GEMV_KINDS[name]).float()
        got = _oracle(name, trans, m, n, alpha, A, lda, x, incx, beta, y, incy)
        len_x, len_y = (n, m) if trans == 0 else (m, n)
        assert_parity(got[::incy], ref[::incy], NAMES[name][1], _scale(len_x, A, x, y, alpha, beta), key)
        if name != "sgemv":
            # one rounding at the end on both sides: the same bits except where the fp32 sums straddle
            # a rounding boundary
            assert float((got[::incy] == ref[::incy]).float().mean()) > 0.98, key
        if beta != 0.0 and incy > 1:
            assert torch.equal(got[1::incy], y.float()[1::incy])


def test_oracle_against_fp64_and_degenerate_cases():
    rng = np.random.default_rng(5)
    A = rng.standard_normal((37, 50)).astype(np.float32)
    for trans, incx, incy in ((0, 1, 1), (1, 2, 3), (0, 3, 2)):
        m, n, lda = 37, 41, 50
        len_x, len_y = (n, m) if trans == 0 else (m, n)
        x = rng.standard_normal(1 + (len_x - 1) * incx).astype(np.float32)
        y = rng.standard_normal(1 + (len_y - 1) * incy).astype(np.float32)
        want = gvo.gemv_fp64(trans, m, n, 1.25, A, lda, x, incx, -0.5, y, incy)
        y0 = y.copy()
        gvo.gemv("sgemv", trans, m, n, 1.25, A, lda, x, incx, -0.5, y, incy)
        np.testing.assert_allclose(y[::incy], want, rtol=1e-5, atol=1e-5)
        for o in range(1, incy):
            np.testing.assert_array_equal(y[o::incy], y0[o::incy])
    y = np.arange(6, dtype=np.float32)
    gvo.gemv("sgemv", 0, 3, 2, 0.0, A, 50, np.ones(2, np.float32), 1, 0.5, y, 2)   # alpha == 0: strided scale
    np.testing.assert_array_equal(y, [0, 1, 1, 3, 2, 5])
    gvo.gemv("sgemv", 0, 3, 2, 0.0, A, 50, np.ones(2, np.float32), 1, 0.0, y, 2)
    np.testing.assert_array_equal(y, [0, 1, 0, 3, 0, 5])
    y = np.arange(6, dtype=np.float32)
    gvo.gemv("sgemv", 0, 0, 2, 1.0, A, 50, np.ones(2, np.float32), 1, 0.0, y, 1)   # empty: untouched
    np.testing.assert_array_equal(y, np.arange(6))
    yh = np.array([np.nan, 7.0], dtype=np.float32)                                 # beta == 0: y not read
    gvo.gemv("hgemv", 0, 1, 2, 1.0, np.array([1.0, 2.0], np.float32), 2, np.array([3.0, 4.0], np.float32), 1, 0.0, yh, 1)
    np.testing.assert_array_equal(yh, [11.0, 7.0])


# ------------------------------------------------------------------------------------ CUDA path
def _run(name, trans, m, n, alpha, beta, pad=0, incx=1, incy=1, seed=0, y_nan=False):
    import flagblas_b200 as fb
    A, lda, x, y = _make(name, trans, m, n, pad, incx, incy, seed, extra_y=3, y_nan=y_nan)
    ref = _oracle(name, trans, m, n, alpha, A, lda, x, incx, beta, y, incy)
    yd = y.to(DEV)
    getattr(fb, name)(trans, m, n, alpha, A.to(DEV), lda, x.to(DEV), incx, beta, yd, incy)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    got = yd.float().cpu()
    len_x = n if trans == 0 else m
    sc = _scale(len_x, A, x, torch.zeros(1) if y_nan else y, alpha, beta)
    assert_parity(got, ref, NAMES[name][1], sc, "%s trans=%d %dx%d a=%g b=%g pad=%d incx=%d incy=%d"
                  % (name, trans, m, n, alpha, beta, pad, incx, incy))
    return got, ref


# general, tiny, ragged, few-rows x long (split over columns), long x few-columns (split over rows),
# the reference's own benchmark squares and an LLM-shaped rectangle
GEMV_SHAPES = [(1, 1), (7, 5), (64, 64), (130, 270), (1000, 300), (300, 1000), (33, 4100), (4100, 33), (1, 9000),
               (9000, 1), (48, 16384), (16384, 48), (1024, 1024), (4096, 4096), (1024, 4096)]


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
@pytest.mark.parametrize("trans", [0, 1])
def test_shapes_alpha_beta(name, trans):
    for i, (m, n) in enumerate(GEMV_SHAPES):
        _run(name, trans, m, n, 1.5, 0.5, seed=i)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
@pytest.mark.parametrize("trans", [0, 1])
def test_strides_padding_and_untouched_elements(name, trans):
    for i, (m, n, pad, incx, incy) in enumerate([(70, 130, 6, 2, 3), (513, 257, 3, 3, 2), (40, 5000, 8, 2, 2),
                                                  (5000, 40, 1, 1, 4), (256, 256, 8, 1, 1)]):
        got, ref = _run(name, trans, m, n, -0.75, 1.0, pad=pad, incx=incx, incy=incy, seed=10 + i)
        # the oracle leaves everything but the strided vector alone; equality of the rest is exact
        len_y = m if trans == 0 else n
        mask = torch.ones_like(got, dtype=torch.bool)
        mask[: 1 + (len_y - 1) * incy : incy] = False
        assert torch.equal(got[mask], ref[mask])


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
@pytest.mark.parametrize("trans", [0, 1])
def test_beta_zero_never_reads_y(name, trans):
    for m, n in [(70, 130), (16, 8192), (8192, 16), (2048, 2048)]:
        got, _ = _run(name, trans, m, n, 2.0, 0.0, incy=2, seed=3, y_nan=True)
        assert not torch.isnan(got).any()


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
@pytest.mark.parametrize("trans", [0, 1])
@pytest.mark.parametrize("beta", [0.0, 0.5, 1.0])
def test_alpha_zero_scales_only_the_strided_vector(name, trans, beta):
    import flagblas_b200 as fb
    m, n, incy = 3, 2, 2
    dt = NAMES[name][0]
    len_x, len_y = (n, m) if trans == 0 else (m, n)
    A = torch.full((m, n), float("nan"), dtype=dt, device=DEV)      # must not be read
    x = torch.full((len_x,), float("nan"), dtype=dt, device=DEV)
    y = torch.arange(len_y * incy, dtype=dt, device=DEV)
    want = y.clone()
    want[::incy] = want[::incy] * beta
    getattr(fb, name)(trans, m, n, 0.0, A, n, x, 1, beta, y, incy)
    torch.cuda.synchronize()
    assert torch.equal(y, want)


@pytest.mark.gpu
def test_empty_and_invalid_arguments():
    import flagblas_b200 as fb
    y = torch.arange(4, dtype=torch.float32, device=DEV)
    A = torch.ones(4, 4, device=DEV)
    x = torch.ones(4, device=DEV)
    fb.sgemv(0, 0, 4, 1.0, A, 4, x, 1, 0.0, y, 1)       # m == 0: nothing happens, even with beta == 0
    fb.sgemv(1, 4, 0, 1.0, A, 4, x, 1, 0.0, y, 1)
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), torch.arange(4, dtype=torch.float32))
    with pytest.raises(AssertionError):
        fb.sgemv(2, 4, 4, 1.0, A, 4, x, 1, 0.0, y, 1)   # CUBLAS_OP_C is not a real-gemv mode
    with pytest.raises(AssertionError):
        fb.sgemv(0, 4, 4, 1.0, A, 3, x, 1, 0.0, y, 1)   # lda < n
    with pytest.raises(AssertionError):
        fb.sgemv(0, 4, 4, 1.0, A, 4, x, 0, 0.0, y, 1)   # incx == 0
    with pytest.raises(AssertionError):
        fb.sgemv(0, 4, 4, 1.0, A, 4, x, 2, 0.0, y, 1)   # x too short for incx
    with pytest.raises(AssertionError):
        fb.hgemv(0, 4, 4, 1.0, A, 4, x, 1, 0.0, y, 1)   # dtype
    lib = fb._lib.lib
    assert lib.fb_gemv(0, 0, 4, 4, 1.0, A.data_ptr(), 3, x.data_ptr(), 1, 0.0, y.data_ptr(), 1, None, 0, None) == -1
    assert lib.fb_gemv(1, 0, 4, 4, 1.0, A.data_ptr(), 4, x.data_ptr(), 1, 0.0, y.data_ptr(), 1, None, 0, None) == -1
    assert lib.fb_gemv(0, 0, 4, 4, 1.0, A.data_ptr(), 4, x.data_ptr(), 1, 0.0, y.data_ptr(), 0, None, 0, None) == -1
    # a split shape without its scratch is refused, not run
    need = lib.fb_gemv_workspace_bytes(0, 0, 4, 1 << 16)
    assert need > 0
    big = torch.ones(4, 1 << 16, device=DEV)
    xs = torch.ones(1 << 16, device=DEV)
    assert lib.fb_gemv(0, 0, 4, 1 << 16, 1.0, big.data_ptr(), 1 << 16, xs.data_ptr(), 1, 0.0, y.data_ptr(), 1, None,
                       0, None) == -2


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
def test_unaligned_base_and_odd_lda(name):
    """A whose rows are not 16-byte aligned takes the element-wise loads: same results."""
    import flagblas_b200 as fb
    dt = NAMES[name][0]
    g = torch.Generator(device="cpu").manual_seed(21)
    m, n, lda = 301, 203, 207
    buf = torch.randn(m * lda + 1, generator=g).to(dt)
    x = torch.randn(max(m, n) + 1, generator=g).to(dt)
    for trans in (0, 1):
        len_x, len_y = (n, m) if trans == 0 else (m, n)
        y = torch.randn(len_y, generator=g).to(dt)
        ref = _oracle(name, trans, m, n, 1.5, buf[1:], lda, x[1:1 + len_x], 1, 0.5, y, 1)
        bd, xd, yd = buf.to(DEV), x.to(DEV), y.to(DEV)
        getattr(fb, name)(trans, m, n, 1.5, bd[1:], lda, xd[1:1 + len_x], 1, 0.5, yd, 1)
        torch.cuda.synchronize()
        assert_parity(yd.float().cpu(), ref, NAMES[name][1], _scale(len_x, buf, x, y, 1.5, 0.5), name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(NAMES))
def test_against_reference_vectors(z, name):
    import flagblas_b200 as fb
    for key, (trans, m, n, lda, incx, incy, alpha, beta), A, x, y in gc.gemv_cases(name):
        ref = gc.unpack(z[key + "_y"], gc.GEMV_KINDS[name]).float()
        yd = y.to(DEV)
        getattr(fb, name)(trans, m, n, alpha, A.to(DEV), lda, x.to(DEV), incx, beta, yd, incy)
        torch.cuda.synchronize()
        got = yd.float().cpu()
        len_x = n if trans == 0 else m
        assert_parity(got[::incy], ref[::incy], NAMES[name][1], _scale(len_x, A, x, y, alpha, beta), key)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["hgemv", "bfgemv", "sgemv"])
@pytest.mark.parametrize("trans", [0, 1])
def test_full_size_properties(name, trans):
    """At the benchmark's size (16384 x 16384) the oracle is not run; the kernel is checked through
    properties instead: reproducibility, an indicator vector picking out one row / column exactly, and
    a column of ones against an fp64 row sum of sampled rows."""
    import flagblas_b200 as fb
    dt = NAMES[name][0]
    m = n = 16384
    g = torch.Generator(device=DEV).manual_seed(7)
    A = torch.randn(m, n, generator=g, device=DEV).to(dt)
    len_x, len_y = (n, m) if trans == 0 else (m, n)
    x = torch.randn(len_x, generator=g, device=DEV).to(dt)
    y1 = torch.zeros(len_y, dtype=dt, device=DEV)
    y2 = torch.full((len_y,), float("nan"), dtype=dt, device=DEV)
    getattr(fb, name)(trans, m, n, 1.0, A, n, x, 1, 0.0, y1, 1)
    getattr(fb, name)(trans, m, n, 1.0, A, n, x, 1, 0.0, y2, 1)
    assert torch.equal(y1, y2)                                   # fixed summation order: bit-reproducible
    e = torch.zeros(len_x, dtype=dt, device=DEV)
    e[12345] = 1.0
    getattr(fb, name)(trans, m, n, 1.0, A, n, e, 1, 0.0, y1, 1)
    pick = A[:, 12345] if trans == 0 else A[12345, :]
    assert torch.equal(y1, pick)                                 # 1 * a + 0 + ... is exact in every type
    rows = torch.tensor([0, 1, 777, 8191, 16383], device=DEV)
    want = (A.index_select(0, rows).double() @ x.double()) if trans == 0 else (A.index_select(1, rows).double().T @ x.double())
    getattr(fb, name)(trans, m, n, 1.0, A, n, x, 1, 0.0, y1, 1)
    torch.cuda.synchronize()
    got = y1.index_select(0, rows).double()
    tol = NAMES[name][1] * (len_x ** 0.5)
    assert float((got - want).abs().max()) <= tol + NAMES[name][1] * float(want.abs().max())
    assert fb.device_status() == 0


# ------------------------------------------------------------------------------------- fp8_gemv
def _fp8_oracle(m, n, lda, incx, incy, ky, alpha, beta, A, x, y):
    yy = y.float().numpy().copy()
    gvo.gemv("fp8_gemv", 1, m, n, alpha, A.float().numpy(), lda, x.float().numpy(), incx, beta, yy, incy, out_kind=ky)
    return torch.from_numpy(yy)


_FP8_TOL = {"fp32": 1e-5, "fp16": 1e-2, "bf16": 1e-2}


def test_fp8_oracle_vs_reference_on_gpu(z):
    for key, (m, n, lda, incx, incy, ky, alpha, beta), A, x, y in gc.fp8_gemv_cases():
        probe = np.concatenate([A.float().numpy().ravel()[:8], x.float().numpy().ravel()[:1]])
        np.testing.assert_array_equal(probe, z[key + "_probe"], err_msg="input generator differs from the fixture's")
        ref = gc.unpack(z[key + "_y"], ky).float()
        got = _fp8_oracle(m, n, lda, incx, incy, ky, alpha, beta, A, x, y)
        assert_parity(got[::incy], ref[::incy], _FP8_TOL[ky], _scale(m, A[:, :n], x[::incx], y[::incy], alpha, beta), key)


@pytest.mark.gpu
def test_fp8_gemv_against_oracle_and_reference_vectors(z):
    import flagblas_b200 as fb
    for key, (m, n, lda, incx, incy, ky, alpha, beta), A, x, y in gc.fp8_gemv_cases():
        yd = y.to(DEV)
        fb.fp8_gemv(1, m, n, alpha, A.to(DEV)[:, :n], lda, x.to(DEV), incx, beta, yd, incy)
        torch.cuda.synchronize()
        got = yd.float().cpu()
        sc = _scale(m, A[:, :n], x[::incx], y[::incy], alpha, beta)
        assert_parity(got, _fp8_oracle(m, n, lda, incx, incy, ky, alpha, beta, A, x, y), _FP8_TOL[ky], sc, key)
        ref = gc.unpack(z[key + "_y"], ky).float()
        assert_parity(got[::incy], ref[::incy], _FP8_TOL[ky], sc, key + " vs reference")
    assert fb.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("ky", ["fp32", "bf16"])
def test_fp8_gemv_shapes_and_edges(fmt, ky):
    import flagblas_b200 as fb
    dt = gc.FP8[fmt]
    g = torch.Generator(device="cpu").manual_seed(41)
    for m, n in [(16, 16), (256, 4096), (8192, 32), (2048, 2048), (4096, 14336)]:
        A = torch.randn(m, n, generator=g).to(dt)
        x = torch.randn(m, generator=g).to(dt)
        y = torch.randn(n, generator=g).to(gc.DTYPES[ky])
        ref = _fp8_oracle(m, n, n, 1, 1, ky, 1.5, 0.5, A, x, y)
        yd = y.to(DEV)
        fb.fp8_gemv(1, m, n, 1.5, A.to(DEV), n, x.to(DEV), 1, 0.5, yd, 1)
        torch.cuda.synchronize()
        assert_parity(yd.float().cpu(), ref, _FP8_TOL[ky], _scale(m, A, x, y, 1.5, 0.5), "fp8 %s %s %dx%d" % (fmt, ky, m, n))
    # beta == 0 never reads y; alpha == 0 only scales; m == 0 does nothing; N form is refused
    yd = torch.full((64,), float("nan"), dtype=gc.DTYPES[ky], device=DEV)
    A = torch.ones(32, 64).to(dt).to(DEV)
    x = torch.ones(32).to(dt).to(DEV)
    fb.fp8_gemv(1, 32, 64, 1.0, A, 64, x, 1, 0.0, yd, 1)
    assert torch.equal(yd.float().cpu(), torch.full((64,), 32.0))
    fb.fp8_gemv(1, 32, 64, 0.0, A, 64, x, 1, 0.5, yd, 1)
    assert torch.equal(yd.float().cpu(), torch.full((64,), 16.0))
    fb.fp8_gemv(1, 0, 64, 1.0, A, 64, x, 1, 0.0, yd, 1)
    assert torch.equal(yd.float().cpu(), torch.full((64,), 16.0))
    with pytest.raises(AssertionError):
        fb.fp8_gemv(0, 32, 64, 1.0, A, 64, x, 1, 0.0, yd, 1)
    with pytest.raises(AssertionError):
        fb.fp8_gemv(1, 32, 60, 1.0, A, 64, x, 1, 0.0, yd, 1)     # n not a multiple of 16
    assert fb.device_status() == 0
