"""Parity of the dense CUDA path (through the flag_blas operator API -> C ABI) against the
CPU oracle on identical seeded inputs, against the reference-made golden vectors, and --
at the benchmark's full sizes -- through size-independent properties.

Tolerances (|got-ref| <= rtol*scale + rtol*|ref|, scale = |alpha|*sqrt(k)*rms(A)*rms(B)):
  fp16 / bf16 1e-2, tf32 1e-3, fp32 (sgemm) 1e-5.
"""
import os

import numpy as np
import pytest
import torch

import flagblas_b200 as fb
from flagblas_b200.ops import CUBLAS_OP_N, CUBLAS_OP_T
from tests.helpers import KINDS, assert_parity, make_dense, oracle_dense, result_scale

pytestmark = pytest.mark.gpu
DEV = "cuda"
TRANS = [(0, 0), (0, 1), (1, 0), (1, 1)]


def _run(kind, ta, tb, m, n, k, alpha, beta, pad=0, seed=0, scale=1.0, c_nan=False):
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, pad=pad, seed=seed, scale=scale, c_nan=c_nan)
    ref = oracle_dense(kind, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
    Ad, Bd, Cd = A.to(DEV), B.to(DEV), C.to(DEV)
    getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, alpha, Ad, lda, Bd, ldb, beta, Cd, ldc)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    got = Cd.float().cpu()
    sc = result_scale(k, A, B, alpha) + abs(beta) * (0.0 if c_nan else 1.0)
    what = "%s ta=%d tb=%d %dx%dx%d a=%g b=%g pad=%d" % (kind, ta, tb, m, n, k, alpha, beta, pad)
    assert_parity(got, ref, KINDS[kind][2], sc, what)
    return got, ref


# shapes: tile-exact, multi-tile, ragged m/n/k, skinny, k tails; (m, n, k)
SHAPES = [(128, 256, 64), (256, 512, 256), (64, 64, 64), (130, 270, 100), (512, 384, 1000), (1, 8, 8), (8, 1, 32),
          (33, 1025, 72), (1000, 72, 4100), (2048, 2048, 512)]


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("ta,tb", TRANS)
def test_shapes_alpha_beta(kind, ta, tb):
    ab = (2.5, 0.5) if kind == "fp32" else (1.5, 0.5)   # the reference tests' pairs
    for i, (m, n, k) in enumerate(SHAPES):
        _run(kind, ta, tb, m, n, k, ab[0], ab[1], seed=i)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("ta,tb", TRANS)
def test_padded_leading_dims_leave_padding_untouched(kind, ta, tb):
    pad = 8 if kind in ("bf16", "fp16") else 4           # keeps rows 16-byte aligned: in-place TMA path
    m, n, k = 200, 328, 136
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, pad=pad, seed=3)
    Cd = C.to(DEV)
    getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, 1.0, A.to(DEV), lda, B.to(DEV), ldb, 1.0, Cd, ldc)
    torch.cuda.synchronize()
    assert torch.equal(Cd.cpu()[:, n:], C[:, n:])
    ref = oracle_dense(kind, ta, tb, m, n, k, 1.0, A, lda, B, ldb, 1.0, C, ldc)
    assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], result_scale(k, A, B, 1.0) + 1.0, "padded %s" % kind)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("ta,tb", TRANS)
def test_unaligned_shapes(kind, ta, tb):
    """Odd sizes with ld == size: rows are not 16-byte aligned (the reference's 511/1023 class)."""
    for (m, n, k) in [(511, 511, 511), (129, 67, 255), (63, 1023, 77)]:
        _run(kind, ta, tb, m, n, k, 1.5, 0.5, seed=7)
    _run(kind, ta, tb, 70, 130, 45, 1.0, 0.0, pad=3, seed=8, c_nan=True)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
def test_misaligned_base_pointers(kind):
    dt = KINDS[kind][0]
    m, n, k = 96, 80, 72
    g = torch.Generator().manual_seed(5)
    bufA = torch.randn(m * k + 8, generator=g).to(dt).to(DEV)
    bufB = torch.randn(k * n + 8, generator=g).to(dt).to(DEV)
    bufC = torch.randn(m * n + 8, generator=g).to(dt).to(DEV)
    for off in (1, 3):
        A, B, C = bufA[off:off + m * k], bufB[off:off + k * n], bufC[off:off + m * n].clone()
        Ch = C.float().cpu().numpy().copy()
        from oracle import gemm_oracle as go
        go.gemm(kind, 0, 0, m, n, k, 1.5, A.float().cpu().numpy(), k, B.float().cpu().numpy(), n, 0.5, Ch, n,
                tf32_mode="trunc")
        Cv = bufC[off:off + m * n]
        getattr(fb, KINDS[kind][1])(0, 0, m, n, k, 1.5, A, k, B, n, 0.5, Cv, n)
        torch.cuda.synchronize()
        assert_parity(Cv.float().cpu(), torch.from_numpy(Ch), KINDS[kind][2],
                      result_scale(k, A.cpu(), B.cpu(), 1.5) + 0.5, "misaligned base %s off=%d" % (kind, off))


# ------------------------------------------------------------------ edge cases (reference tests/test_sgemm.py:148-245)
@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
def test_alpha_zero_scales_c(kind):
    A, lda, B, ldb, C, ldc = make_dense(kind, 0, 0, 64, 64, 64, seed=1)
    Cd = C.to(DEV)
    getattr(fb, KINDS[kind][1])(0, 0, 64, 64, 64, 0.0, A.to(DEV), lda, B.to(DEV), ldb, 0.5, Cd, ldc)
    ref = oracle_dense(kind, 0, 0, 64, 64, 64, 0.0, A, lda, B, ldb, 0.5, C, ldc)
    assert torch.equal(Cd.float().cpu(), ref)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("ta,tb", TRANS)
def test_beta_zero_never_reads_c(kind, ta, tb):
    got_nan, _ = _run(kind, ta, tb, 192, 320, 96, 2.5, 0.0, seed=2, c_nan=True)
    assert not torch.isnan(got_nan).any()
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, 192, 320, 96, seed=2)
    Cz = torch.zeros_like(C).to(DEV)
    getattr(fb, KINDS[kind][1])(ta, tb, 192, 320, 96, 2.5, A.to(DEV), lda, B.to(DEV), ldb, 0.0, Cz, ldc)
    assert torch.equal(Cz.float().cpu(), got_nan)   # NaN-filled and zero-filled C give identical bits


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
@pytest.mark.parametrize("m,n,k", [(0, 64, 64), (64, 0, 64), (64, 64, 0)])
def test_empty_dims_scale_whole_c(kind, m, n, k):
    dt = KINDS[kind][0]
    g = torch.Generator().manual_seed(4)
    A = torch.randn(max(m, 1) * max(k, 1), generator=g).to(dt)
    B = torch.randn(max(k, 1) * max(n, 1), generator=g).to(dt)
    C = torch.randn(max(m, 1), max(n, 1), generator=g).to(dt)   # e.g. (1 x 64) for m == 0
    Cd = C.to(DEV)
    getattr(fb, KINDS[kind][1])(0, 0, m, n, k, 2.5, A.to(DEV), max(k, 1), B.to(DEV), max(n, 1), 0.5, Cd, max(n, 1))
    ref = oracle_dense(kind, 0, 0, m, n, k, 2.5, A, max(k, 1), B, max(n, 1), 0.5, C, max(n, 1))
    assert torch.equal(Cd.float().cpu(), ref)
    Cd = C.to(DEV)
    getattr(fb, KINDS[kind][1])(0, 0, m, n, k, 2.5, A.to(DEV), max(k, 1), B.to(DEV), max(n, 1), 0.0, Cd, max(n, 1))
    assert torch.count_nonzero(Cd) == 0


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32", "fp32"])
def test_alpha_beta_pairs_and_tensor_scalars(kind):
    for alpha, beta in [(1.0, 0.0), (0.0, 1.0), (1.0, 1.0), (-1.0, 0.5), (2.5, -0.5)]:
        _run(kind, 0, 0, 256, 256, 256, alpha, beta, seed=9)
    A, lda, B, ldb, C, ldc = make_dense(kind, 0, 1, 128, 128, 128, seed=10)
    C1, C2 = C.to(DEV), C.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    op(0, 1, 128, 128, 128, 1.5, A.to(DEV), lda, B.to(DEV), ldb, 0.5, C1, ldc)
    op(0, 1, 128, 128, 128, torch.tensor(1.5, device=DEV), A.to(DEV), lda, B.to(DEV), ldb, torch.tensor(0.5), C2, ldc)
    assert torch.equal(C1, C2)


# ------------------------------------------------------------------ reference-made golden vectors on the GPU
@pytest.mark.parametrize("ta,tb", TRANS)
@pytest.mark.parametrize("m,n,k,pad", [
    (2048, 2048, 1024, 0),    # 256 tiles of 128 x 128
    (1920, 1666, 1000, 0),    # ragged edge tiles, k not a multiple of the 16-deep slice
    (1600, 2000, 520, 4),     # padded leading dimensions
    (1664, 1792, 768, 3),     # odd leading dimensions: the register-staged kernel instead of the cp.async pipeline
])
def test_sgemm_large_tiles_every_layout(ta, tb, m, n, k, pad, monkeypatch):
    """IEEE fp32 with 128 x 128 tiles in all four layouts (NT stores B's slices pair-interleaved for packed FMAs;
    FLAGBLAS_B200_SGEMM_NT_PAIRS=0 keeps plain tiles and scalar FMAs): both against the fp64 product."""
    A, lda, B, ldb, C, ldc = make_dense("fp32", ta, tb, m, n, k, pad=pad, seed=41, scale=0.5)
    Ad, Bd = A.to(DEV), B.to(DEV)
    opA = (Ad[:, :m].t() if ta else Ad[:, :k]).double()
    opB = (Bd[:, :k].t() if tb else Bd[:, :n]).double()
    ref = (1.25 * (opA @ opB) + 0.5 * C.to(DEV)[:, :n].double()).float().cpu()
    sc = result_scale(k, A, B, 1.25) + 0.5
    for pairs in ("1", "0"):
        monkeypatch.setenv("FLAGBLAS_B200_SGEMM_NT_PAIRS", pairs)
        fb.reload_env()
        Cd = C.to(DEV)
        fb.sgemm(ta, tb, m, n, k, 1.25, Ad, lda, Bd, ldb, 0.5, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert_parity(Cd[:, :n].float().cpu(), ref, KINDS["fp32"][2], sc, "sgemm pairs=%s ta=%d tb=%d %dx%dx%d" % (pairs, ta, tb, m, n, k))
        if pad:
            assert torch.equal(Cd[:, n:].cpu(), C[:, n:]), "padding columns of C were touched"


@pytest.mark.parametrize("kind", ["fp32", "fp16"])
def test_golden_dense_on_gpu(golden_dir, kind):
    z = np.load(os.path.join(golden_dir, "dense_%s.npz" % kind))
    dt = KINDS[kind][0]
    for key in sorted(k[:-2] for k in z.files if k.endswith("_p")):
        ta, tb, m, n, k, lda, ldb, ldc, alpha, beta = z[key + "_p"]
        ta, tb, m, n, k, lda, ldb, ldc = (int(v) for v in (ta, tb, m, n, k, lda, ldb, ldc))
        A = torch.from_numpy(z[key + "_A"]).to(dt).to(DEV)
        B = torch.from_numpy(z[key + "_B"]).to(dt).to(DEV)
        C = torch.from_numpy(z[key + "_C0"]).to(dt).to(DEV)
        getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, float(alpha), A, lda, B, ldb, float(beta), C, ldc)
        ref = torch.from_numpy(z[key + "_C"])
        got = C.float().cpu()
        assert torch.equal(got[:, n:], ref[:, n:])
        assert_parity(got[:, :n], ref[:, :n], KINDS[kind][2], result_scale(k, A.cpu(), B.cpu(), alpha) + abs(beta),
                      "golden %s %s" % (kind, key))


def test_golden_config1_sgemm512(golden_dir):
    z = np.load(os.path.join(golden_dir, "config1_sgemm512.npz"))
    g = torch.Generator(device="cpu").manual_seed(0)
    A = torch.rand(512, 512, generator=g) * 2 - 1
    B = torch.rand(512, 512, generator=g) * 2 - 1
    C = torch.full((512, 512), float("nan"), device=DEV)
    fb.sgemm(CUBLAS_OP_N, CUBLAS_OP_N, 512, 512, 512, 1.0, A.to(DEV), 512, B.to(DEV), 512, 0.0, C, 512)
    got = C.cpu()
    ref = torch.from_numpy(z["C_sub"])
    assert_parity(got[::4, ::4], ref, 1e-5, result_scale(512, A, B, 1.0), "config1")
    assert abs(float(got.double().sum()) - float(z["C_sum"])) < 1e-2


# ------------------------------------------------------------------ full benchmark sizes, size-independent properties
def _cublas(kind, ta, tb, A, B):
    opA = A.t() if ta else A
    opB = B.t() if tb else B
    return (opA.float() @ opB.float()) if kind != "fp32" else opA @ opB


@pytest.mark.parametrize("cfg", ["hgemm_8192_nn", "bfgemm_mlp_nt", "tf32gemm_skinny_tn", "tf32gemm_4096_tn", "tf32gemm_16384_tn"])
def test_full_size_properties(cfg):
    """The benchmark workloads at full size, where the CPU oracle cannot finish: (1) whole rows and columns against
    an fp64 product of the same (for TF32: truncated) operands, (2) exact linearity in alpha, (3) NaN-filled C is
    never read when beta == 0, (4) the whole result against cuBLAS through torch, block of rows by block of rows."""
    torch.backends.cuda.matmul.allow_tf32 = False
    uniform = False     # operands N(0, 1) * s, or U(-1, 1)
    if cfg == "hgemm_8192_nn":
        kind, ta, tb, m, n, k, alpha, beta, sa, sb, sc0, seed = "fp16", 0, 0, 8192, 8192, 8192, 1.0, 0.0, 0.05, 0.05, 0.02, 1
    elif cfg == "bfgemm_mlp_nt":
        kind, ta, tb, m, n, k, alpha, beta, sa, sb, sc0, seed = "bf16", 0, 1, 16384, 14336, 4096, 1.0, 1.0, 1.0, 0.02, 0.02, 2
    else:
        mm = {"tf32gemm_skinny_tn": 64, "tf32gemm_4096_tn": 4096, "tf32gemm_16384_tn": 16384}[cfg]
        nk = 4096 if cfg == "tf32gemm_4096_tn" else 16384
        kind, ta, tb, m, n, k, alpha, beta, sa, sb, sc0, seed = "tf32", 1, 0, mm, nk, nk, 1.5, 0.5, 0.577, 0.577, 0.577, 4
        uniform = True
    dt, opname, rtol = KINDS[kind]
    op = getattr(fb, opname)
    g = torch.Generator(device=DEV).manual_seed(seed)

    def draw(shape, s):
        if uniform:
            return torch.rand(shape, generator=g, device=DEV) * 2 - 1
        return (torch.randn(shape, generator=g, device=DEV) * s).to(dt)

    A = draw((k, m) if ta else (m, k), sa)
    B = draw((n, k) if tb else (k, n), sb)
    C0 = draw((m, n), sc0)
    if beta == 0.0:
        C0.fill_(float("nan"))
    C = C0.clone()
    op(ta, tb, m, n, k, alpha, A, A.shape[1], B, B.shape[1], beta, C, n)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert not torch.isnan(C).any()
    # (1) sampled rows and columns against fp64 (formed on the GPU by cuBLAS's dgemm: a checker, not the product)
    rows = torch.tensor(sorted(r for r in {0, 1, 127, 128, m // 2 + 3, m - 1} if r < m), device=DEV)
    cols = torch.tensor(sorted(c for c in {0, 255, 256, n // 2 + 5, n - 1} if c < n), device=DEV)
    trunc = (lambda x: (x.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)) if kind == "tf32" else (lambda x: x)
    a_rows = trunc(A[:, rows].t() if ta else A[rows]).double()            # [rows, k]
    b_cols = trunc(B[cols].t() if tb else B[:, cols]).double()            # [k, cols]
    sc = abs(alpha) * (k ** 0.5) * sa * sb + abs(beta) * sc0
    ref_rows = torch.empty(len(rows), n, dtype=torch.float64, device=DEV)
    ref_cols = torch.empty(m, len(cols), dtype=torch.float64, device=DEV)
    step = 2048
    for j in range(0, n, step):      # operand blocks are widened to fp64 piece by piece
        bj = trunc(B[j:j + step].t() if tb else B[:, j:j + step]).double()
        ref_rows[:, j:j + step] = alpha * (a_rows @ bj)
    for i in range(0, m, step):
        ai = trunc(A[:, i:i + step].t() if ta else A[i:i + step]).double()
        ref_cols[i:i + step] = alpha * (ai @ b_cols)
    if beta != 0.0:
        ref_rows += beta * C0[rows].double()
        ref_cols += beta * C0[:, cols].double()
    assert_parity(C[rows].float().cpu(), ref_rows.float().cpu(), rtol, sc, cfg + " rows")
    assert_parity(C[:, cols].float().cpu(), ref_cols.float().cpu(), rtol, sc, cfg + " cols")
    del ref_rows, ref_cols, a_rows, b_cols
    # (2) linearity: doubling alpha (beta = 0) doubles the result -- exactly for normal numbers
    # (power-of-two scaling commutes with rounding); fp16 subnormals may differ by one step (2^-24)
    C1 = torch.empty_like(C)
    op(ta, tb, m, n, k, 1.0, A, A.shape[1], B, B.shape[1], 0.0, C1, n)
    op(ta, tb, m, n, k, 2.0, A, A.shape[1], B, B.shape[1], 0.0, C, n)
    lin_tol = 2.0 ** -23 if kind == "fp16" else 0.0
    for i in range(0, m, step):
        assert float((C1[i:i + step].float() * 2.0 - C[i:i + step].float()).abs().max()) <= lin_tol
    # (4) independent cross-check of the whole result: cuBLAS through torch on the same data, by row blocks
    opB = (B.t() if tb else B)
    opB = opB.float() if kind != "tf32" else opB
    bound_abs = 2 * rtol * (k ** 0.5) * sa * sb
    for i in range(0, m, step):
        ai = (A[:, i:i + step].t() if ta else A[i:i + step])
        refc = (ai.float() if kind != "tf32" else ai) @ opB
        d = (C1[i:i + step].float() - refc).abs().max().item()
        assert d <= bound_abs + rtol * refc.abs().max().item(), (cfg, i, d)


@pytest.mark.parametrize("kind,ta,tb,beta", [("bf16", 0, 1, 0.5), ("fp16", 0, 0, 0.0), ("tf32", 1, 0, 0.5), ("fp32", 0, 0, 0.0)])
def test_gemm_from_host_matches_the_operator(kind, ta, tb, beta):
    """Host-memory entry: row blocks streamed over three CUDA streams (transa = N) or the plain
    copy / compute / copy sequence (transa = T) must give the operator's result: to the last bit where a row block
    takes the same tile plan as the whole call, otherwise (a row block may be small enough for a split of k, which
    adds in another order) within the operator's own tolerance; untouched padding stays untouched."""
    from flagblas_b200 import host
    m, n, k = 2304, 640, 512
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, pad=8, seed=5)
    name = KINDS[kind][1]
    Cd = C.to(DEV)
    getattr(fb, name)(ta, tb, m, n, k, 1.5, A.to(DEV), lda, B.to(DEV), ldb, beta, Cd, ldc)
    torch.cuda.synchronize()
    hA, hB, hC = A.pin_memory(), B.pin_memory(), C.clone().pin_memory()
    dA, dB, dC = torch.empty_like(A, device=DEV), torch.empty_like(B, device=DEV), torch.full_like(C, float("nan"), device=DEV)
    for _ in range(2):   # twice: the second call reuses streams and scratch
        hC.copy_(C)
        host.gemm_from_host(name, ta, tb, m, n, k, 1.5, hA, lda, hB, ldb, beta, hC, ldc, dA, dB, dC, chunks=4)
        torch.cuda.current_stream().synchronize()
        assert_parity(hC[:, :n].float(), Cd.cpu()[:, :n].float(), KINDS[kind][2], result_scale(k, A, B, 1.5) + abs(beta),
                      "from host %s" % kind)
        if beta != 0.0:
            assert torch.equal(hC[:, n:], Cd.cpu()[:, n:])
    assert fb.device_status() == 0


def test_cuda_graph_capture_and_replay():
    """A launch-bound sequence (small GEMM, matrix-vector product, grouped GEMM) captured once in a CUDA graph
    and replayed on new input data gives what eager calls give."""
    g = torch.Generator(device="cpu").manual_seed(77)
    m, n, k = 256, 384, 320
    A = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    B = torch.randn(k, n, generator=g).bfloat16().to(DEV)
    C = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    x = torch.randn(n, generator=g).bfloat16().to(DEV)
    y = torch.zeros(m, dtype=torch.bfloat16, device=DEV)
    ms, K, N = [100, 0, 156], 320, 128
    Bg = (torch.randn(3 * K, N, generator=g) / 16).bfloat16().to(DEV)
    O = torch.zeros(sum(ms), N, dtype=torch.bfloat16, device=DEV)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=DEV)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    starts = [0, 100, 100]
    ga = (O, i64([A.data_ptr() + s * K * 2 for s in starts]), i64([Bg.data_ptr() + e * K * N * 2 for e in range(3)]),
          i64([O.data_ptr() + s * N * 2 for s in starts]), i64([O.data_ptr() + s * N * 2 for s in starts]), i32(ms),
          i32([N] * 3), i32([K] * 3), i32([K] * 3), i32([N] * 3), i32([N] * 3), 3, sum(ms), N, K, 1.0, 0.0)

    def run():
        fb.bfgemm(0, 0, m, n, k, 1.0, A, k, B, n, 0.0, C, n)
        fb.bfgemv(0, m, n, 1.0, C, n, x, 1, 0.0, y, 1)         # consumes the GEMM's output
        fb.group_bfgemm(*ga)

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        run()                                                   # first call on this stream: outside any capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        run()
    A.copy_(torch.randn(m, k, generator=g).bfloat16())         # new data, same buffers
    x.copy_(torch.randn(n, generator=g).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    got = (C.clone(), y.clone(), O.clone())
    run()
    torch.cuda.synchronize()
    assert torch.equal(got[0], C) and torch.equal(got[1], y) and torch.equal(got[2], O)
    assert float(C.float().abs().max()) > 0 and float(O.float().abs().max()) > 0
    assert fb.device_status() == 0
