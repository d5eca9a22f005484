"""Seeded inputs of the GPU golden vectors, shared by the generator (``make_golden_gpu.py``) and the
tests that consume ``gpu_reference.npz``.  Only the reference's outputs are stored in the fixture; the
inputs are regenerated from these seeds (torch's CPU generator), and a few input elements are stored
alongside to detect a generator mismatch."""
import torch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "tf32": torch.float32}
DENSE_AB = {"bf16": (1.5, 0.5), "fp16": (1.5, 0.5), "fp32": (2.5, 0.5)}
DENSE_SHAPES = {"bf16": ((96, 80, 72, 0), (70, 130, 45, 8)), "fp16": ((70, 130, 45, 8),), "fp32": ((70, 130, 45, 4),)}
GROUP_MS, GROUP_K, GROUP_N = [5, 0, 70, 33, 100], 256, 192
GROUP_AB = {"ab": (1.5, 0.5), "b0": (1.0, 0.0)}


def dense_cases(kind):
    """Yields (key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C) as CPU tensors."""
    dt = DTYPES[kind]
    gen = torch.Generator(device="cpu").manual_seed(31)
    alpha, beta = DENSE_AB[kind]
    for ta in (0, 1):
        for tb in (0, 1):
            for ci, (m, n, k, pad) in enumerate(DENSE_SHAPES[kind]):
                lda, ldb, ldc = (m if ta else k) + pad, (k if tb else n) + pad, n + pad
                A = torch.randn((k if ta else m), lda, generator=gen).to(dt)
                B = torch.randn((n if tb else k), ldb, generator=gen).to(dt)
                C = torch.randn(m, ldc, generator=gen).to(dt)
                yield "dense_%s_t%d%d_c%d" % (kind, ta, tb, ci), (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C


def group_case(kind, tag):
    """(ms, K, N, alpha, beta, A [sum m, K], B [E*K, N], C [sum m, N]) as CPU tensors."""
    dt = DTYPES[kind]
    gen = torch.Generator(device="cpu").manual_seed(33)
    E = len(GROUP_MS)
    A = torch.randn(sum(GROUP_MS), GROUP_K, generator=gen).to(dt)
    B = (torch.randn(E * GROUP_K, GROUP_N, generator=gen) * GROUP_K ** -0.5).to(dt)
    C = torch.randn(sum(GROUP_MS), GROUP_N, generator=gen).to(dt)
    alpha, beta = GROUP_AB[tag]
    return GROUP_MS, GROUP_K, GROUP_N, alpha, beta, A, B, C


def tf32_probe():
    """All-positive fp32 inputs: truncating the operands to TF32 shows up as a ~7e-4 shrink of every
    output, rounding them to nearest does not."""
    gen = torch.Generator(device="cpu").manual_seed(34)
    m, n, k = 128, 128, 2048
    return m, n, k, torch.rand(m, k, generator=gen) + 0.5, torch.rand(n, k, generator=gen) + 0.5


def group_mm_case():
    gen = torch.Generator(device="cpu").manual_seed(35)
    A = torch.randn(216, 128, generator=gen).bfloat16()
    B = (torch.randn(4, 128, 96, generator=gen) / 11).bfloat16()
    offs = torch.tensor([20, 20, 150, 216], dtype=torch.int32)
    return A, B, offs


GEMV_KINDS = {"sgemv": "fp32", "hgemv": "fp16", "bfgemv": "bf16"}
# (m, n, lda - n, incx, incy, alpha, beta): general, strided, the reference's split-K shapes
# (m <= 64 and n >= 4096; the mirrored one for trans = T), its small power-of-two-n kernel, beta == 0.
GEMV_SHAPES = ((70, 130, 6, 1, 1, 1.5, 0.5), (33, 47, 0, 2, 3, -0.75, 1.0), (48, 5000, 8, 1, 1, 1.5, 0.5),
               (4200, 40, 0, 1, 1, 1.5, 0.5), (100, 16, 0, 1, 1, 2.0, 0.0))


def gemv_cases(name):
    """Yields (key, (trans, m, n, lda, incx, incy, alpha, beta), A, x, y) as CPU tensors."""
    dt = DTYPES[GEMV_KINDS[name]]
    gen = torch.Generator(device="cpu").manual_seed(36)
    for trans in (0, 1):
        for ci, (m, n, pad, incx, incy, alpha, beta) in enumerate(GEMV_SHAPES):
            lda = n + pad
            len_x, len_y = (n, m) if trans == 0 else (m, n)
            A = torch.randn(m, lda, generator=gen).to(dt)
            x = torch.randn(1 + (len_x - 1) * incx, generator=gen).to(dt)
            y = torch.randn(1 + (len_y - 1) * incy, generator=gen).to(dt)
            yield "gemv_%s_t%d_c%d" % (name, trans, ci), (trans, m, n, lda, incx, incy, alpha, beta), A, x, y


FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
# (m, n, lda - n, incx, incy, A format, x format, y kind, alpha, beta): plain, the reference's split-K
# shape (n <= 64 and m >= 4096), e5m2 with fp16 output, mixed formats with strides.
FP8_GEMV_SHAPES = ((256, 128, 0, 1, 1, "e4m3", "e4m3", "fp32", 1.5, 0.5), (4112, 48, 16, 1, 1, "e4m3", "e4m3", "bf16", 1.0, 0.0),
                   (512, 1024, 0, 1, 1, "e5m2", "e5m2", "fp16", 2.0, 1.0), (320, 208, 32, 2, 2, "e4m3", "e5m2", "fp32", -0.5, 0.25))


def fp8_gemv_cases():
    """Yields (key, (m, n, lda, incx, incy, y kind, alpha, beta), A, x, y) as CPU tensors (A, x in FP8)."""
    gen = torch.Generator(device="cpu").manual_seed(37)
    for ci, (m, n, pad, incx, incy, fa, fx, ky, alpha, beta) in enumerate(FP8_GEMV_SHAPES):
        lda = n + pad
        A = torch.randn(m, lda, generator=gen).to(FP8[fa])
        x = torch.randn(1 + (m - 1) * incx, generator=gen).to(FP8[fx])
        y = torch.randn(1 + (n - 1) * incy, generator=gen).to(DTYPES[ky])
        yield "fp8gemv_c%d" % ci, (m, n, lda, incx, incy, ky, alpha, beta), A, x, y


XGEMM = {"dgemm": ("fp64", torch.float64, 2.5, 0.5), "cgemm": ("c64", torch.complex64, 2.5 + 0.5j, 0.5 - 0.25j),
         "zgemm": ("c128", torch.complex128, 2.5 + 0.5j, 0.5 - 0.25j)}
XGEMM_SHAPES = ((40, 72, 45, 3), (33, 17, 64, 0))
XGEMM_OPS = {False: ((0, 0), (0, 1), (1, 0), (1, 1)), True: ((0, 0), (1, 0), (0, 2), (2, 1), (2, 2))}


def xgemm_cases(name):
    """Yields (key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C) as CPU tensors."""
    kind, dt, alpha, beta = XGEMM[name]
    gen = torch.Generator(device="cpu").manual_seed(38)
    for ta, tb in XGEMM_OPS[dt.is_complex]:
        for ci, (m, n, k, pad) in enumerate(XGEMM_SHAPES):
            lda, ldb, ldc = (m if ta else k) + pad, (k if tb else n) + pad, n + pad
            A = torch.randn((k if ta else m), lda, generator=gen, dtype=dt)
            B = torch.randn((n if tb else k), ldb, generator=gen, dtype=dt)
            C = torch.randn(m, ldc, generator=gen, dtype=dt)
            yield "%s_t%d%d_c%d" % (name, ta, tb, ci), (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C


TRMM = {"strmm": ("fp32", torch.float32, 1.5), "dtrmm": ("fp64", torch.float64, 1.5),
        "ctrmm": ("c64", torch.complex64, 1.5 - 0.5j), "ztrmm": ("c128", torch.complex128, 1.5 - 0.5j)}
# (side, uplo, trans, diag, m, n, pad)
TRMM_MODES = ((0, 0, 0, 0, 70, 40, 2), (0, 1, 1, 1, 70, 40, 0), (1, 1, 0, 0, 36, 72, 3), (1, 0, 1, 1, 36, 72, 0),
              (0, 1, 2, 0, 33, 20, 0), (1, 0, 2, 1, 20, 33, 1))


def trmm_cases(name):
    """Yields (key, (side, uplo, trans, diag, m, n, lda, ldb, ldc, alpha), A, B, C) as CPU tensors."""
    kind, dt, alpha = TRMM[name]
    gen = torch.Generator(device="cpu").manual_seed(39)
    for ci, (side, uplo, trans, diag, m, n, pad) in enumerate(TRMM_MODES):
        if trans == 2 and not dt.is_complex:
            continue
        k = m if side == 0 else n
        lda, ldb, ldc = k + pad, n + pad, n + pad
        A = torch.randn(k, lda, generator=gen, dtype=dt)
        B = torch.randn(m, ldb, generator=gen, dtype=dt)
        C = torch.randn(m, ldc, generator=gen, dtype=dt)
        yield "%s_c%d" % (name, ci), (side, uplo, trans, diag, m, n, lda, ldb, ldc, alpha), A, B, C


# ---------------------------------------------------------------- the benchmark workloads at full size
# name: (kind, transa, transb, m, n, k, alpha, beta, seed); inputs as the benchmark states them.
FULL_SIZE = {
    "hgemm_8192_nn": ("fp16", 0, 0, 8192, 8192, 8192, 1.0, 0.0, 1),
    "bfgemm_mlp_nt": ("bf16", 0, 1, 16384, 14336, 4096, 1.0, 1.0, 2),
    "tf32gemm_16384_tn": ("tf32", 1, 0, 16384, 16384, 16384, 1.5, 0.5, 4),
    "tf32gemm_skinny_tn": ("tf32", 1, 0, 64, 16384, 16384, 1.5, 0.5, 4),
}
MOE = {"experts": 64, "k": 4096, "n": 1536, "tokens": 32768, "zipf": 1.2, "seed": 3}


def full_size_dense(name):
    """(kind, ta, tb, m, n, k, alpha, beta, A, B, C) of a full-size dense workload, CPU tensors in storage layout:
    fp16 8192^3 with N(0,1)*0.05 operands; the bf16 MLP shape with A ~ N(0,1), B and C ~ N(0,0.02); the TF32 shapes
    with U(-1,1) operands and C."""
    kind, ta, tb, m, n, k, alpha, beta, seed = FULL_SIZE[name]
    dt = DTYPES[kind]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    a_shape, b_shape = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
    if kind == "fp16":
        A = (torch.randn(a_shape, generator=gen) * 0.05).to(dt)
        B = (torch.randn(b_shape, generator=gen) * 0.05).to(dt)
        C = torch.zeros(m, n, dtype=dt)
    elif kind == "bf16":
        A = torch.randn(a_shape, generator=gen).to(dt)
        B = (torch.randn(b_shape, generator=gen) * 0.02).to(dt)
        C = (torch.randn(m, n, generator=gen) * 0.02).to(dt)
    else:
        A = torch.rand(a_shape, generator=gen) * 2 - 1
        B = torch.rand(b_shape, generator=gen) * 2 - 1
        C = torch.rand(m, n, generator=gen) * 2 - 1
    return kind, ta, tb, m, n, k, alpha, beta, A, B, C


def sample_rows_cols(m, n, count=8):
    """Rows and columns of a full-size result that the fixture keeps: both edges, tile seams and a spread."""
    def pick(size):
        want = [0, 127, 128, 256, size // 3 + 5, size // 2 + 3, (2 * size) // 3 + 7, size - 1]
        return sorted({v for v in want if 0 <= v < size})[:count]
    return pick(m), pick(n)


def moe_case():
    """(ms, K, N, A [tokens, K], B [E * K, N]) of the grouped MoE workload: token counts drawn from
    Multinomial(tokens, Zipf(1.2) weights over the experts), zeros allowed; A ~ N(0,1), B ~ N(0,0.02), bf16."""
    E, K, N, T = MOE["experts"], MOE["k"], MOE["n"], MOE["tokens"]
    gen = torch.Generator(device="cpu").manual_seed(MOE["seed"])
    w = torch.arange(1, E + 1, dtype=torch.float64) ** -MOE["zipf"]
    ms = torch.multinomial(w / w.sum(), T, replacement=True, generator=gen).bincount(minlength=E).tolist()
    A = torch.randn(T, K, generator=gen).bfloat16()
    B = (torch.randn(E * K, N, generator=gen) * 0.02).bfloat16()
    return ms, K, N, A, B


MOE_COLS = [0, 255, 256, 1535]


def pack(t):
    """Storage-exact numpy form: 16-bit types as their bit patterns, fp32 as is."""
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def unpack(a, kind):
    t = torch.from_numpy(a)
    if kind in ("bf16", "fp16"):
        return t.view(DTYPES[kind])
    return t
