"""The dense kernel's alternative configurations (single-CTA tiles, 2-D copies, one or two k-slabs per stage,
narrow and 512-wide tiles with the B stage fetched by one copy or two, streaming stores) must compute the same
results as the default plan."""
import pytest
import torch

import flagblas_b200 as fb
from tests.helpers import KINDS, assert_parity, make_dense, oracle_dense, result_scale

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("env", [{"FLAGBLAS_B200_PAIR": "0"}, {"FLAGBLAS_B200_TMA3D": "0"}, {"FLAGBLAS_B200_KS": "1"},
                                 {"FLAGBLAS_B200_BLOCK_N": "128"}, {"FLAGBLAS_B200_PAIR": "0", "FLAGBLAS_B200_BLOCK_N": "64"},
                                 {"FLAGBLAS_B200_STAGES": "2"}, {"FLAGBLAS_B200_GROUP_M": "3"},
                                 {"FLAGBLAS_B200_BLOCK_N": "512"}, {"FLAGBLAS_B200_BLOCK_N": "512", "FLAGBLAS_B200_KS": "2"},
                                 {"FLAGBLAS_B200_BLOCK_N": "512", "FLAGBLAS_B200_WIDE_MERGED": "0"},
                                 {"FLAGBLAS_B200_BLOCK_N": "512", "FLAGBLAS_B200_WIDE_MERGED": "0", "FLAGBLAS_B200_KS": "1"},
                                 {"FLAGBLAS_B200_BLOCK_N": "512", "FLAGBLAS_B200_C_STREAMING": "1"},
                                 {"FLAGBLAS_B200_C_STREAMING": "1"}])
@pytest.mark.parametrize("kind", ["bf16", "tf32"])
def test_dense_plan_variants(env, kind, monkeypatch):
    for k, v in env.items():
        monkeypatch.setenv(k, v)
        fb.reload_env()
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
        m, n, k = 640, 896, 448
        A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=21)
        ref = oracle_dense(kind, ta, tb, m, n, k, 1.5, A, lda, B, ldb, 0.5, C, ldc)
        Cd = C.to(DEV)
        getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, 1.5, A.to(DEV), lda, B.to(DEV), ldb, 0.5, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], result_scale(k, A, B, 1.5) + 0.5, "%s %s ta=%d tb=%d" % (kind, env, ta, tb))


@pytest.mark.parametrize("kind,ta,tb,m,n,k", [
    ("bf16", 0, 1, 1024, 1024, 4096),    # 16 pair tiles over all workers: every tile split ~5 ways
    ("fp16", 0, 0, 4096, 4096, 1024),    # 3 whole waves + a 34-tile tail
    ("bf16", 1, 0, 2304, 2048, 2048),    # ragged tail
    ("tf32", 1, 0, 64, 8192, 8192),      # skinny: 64 single-CTA tiles spread over all SMs
    ("tf32", 0, 1, 1000, 1536, 2000),    # edge tiles inside a split tile
    ("bf16", 0, 0, 130, 4100, 6144),     # single-CTA tiles (m <= 128 ... two row blocks), ragged n
    ("bf16", 0, 1, 4096, 4096, 4096),    # 3 whole waves + 34 tail tiles, two workers per tail tile
    ("fp16", 0, 0, 2560, 4096, 4096),    # 2 whole waves + 12 tail tiles, four workers per tail tile
    ("tf32", 1, 0, 4096, 4096, 2048),    # the same tail in TF32
    ("bf16", 1, 1, 4000, 4000, 4160),    # ragged edge tiles, last k stage half full
    ("bf16", 0, 1, 1024, 1536, 4096),    # 24 pair tiles and no whole wave: three sharers, each finishing a part of the columns
    ("fp16", 0, 0, 1000, 1500, 4104),    # the same with ragged edges
    ("bf16", 0, 1, 256, 8192, 8192),     # 32 pair tiles: two sharers, owner and contributor
    ("tf32", 1, 0, 512, 4096, 4096),     # TF32, 32 pair tiles
])
@pytest.mark.parametrize("beta", [0.5, 0.0])
def test_stream_k_tail(kind, ta, tb, m, n, k, beta, monkeypatch):
    """The stream-K tail (FLAGBLAS_B200_STREAMK=0 switches it off): when the last wave of tiles is at most half
    full and k is long, each tail tile is shared by 2-4 workers (partial sums parked in the workspace; two sharers:
    the tile's owner adds the other's; more: every sharer finishes a part of the columns).  beta = 0 takes the
    epilogue that stores through TMA.  Same tolerance as every other dense test, and close agreement with whole tiles."""
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=31, scale=0.25)
    Ad, Bd = A.to(DEV), B.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    outs = {}
    for sk in ("1", "0"):
        monkeypatch.setenv("FLAGBLAS_B200_STREAMK", sk)
        fb.reload_env()
        Cd = C.to(DEV)
        op(ta, tb, m, n, k, 1.5, Ad, lda, Bd, ldb, beta, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        outs[sk] = Cd.float().cpu()
    sc = result_scale(k, A, B, 1.5) + beta
    # both schedules against fp64 on the GPU-resident data (the numpy oracle is too slow at these sizes)
    opA = (Ad.t() if ta else Ad).double()
    opB = (Bd.t() if tb else Bd).double()
    if kind == "tf32":
        trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
        opA, opB = trunc(opA), trunc(opB)
    ref = (1.5 * (opA @ opB) + beta * C.to(DEV).double()).float().cpu()
    for sk in ("1", "0"):
        assert_parity(outs[sk], ref, KINDS[kind][2], sc, "stream-k=%s %s %dx%dx%d beta=%g" % (sk, kind, m, n, k, beta))
    # different summation order: the two schedules may differ by a rounding step of the output type
    assert_parity(outs["1"], outs["0"], KINDS[kind][2], sc, "stream-k vs whole tiles")


def test_stream_k_calls_on_two_streams():
    """Calls whose tiles share their k ranges, issued alternately on two streams: the library orders a stream-K
    launch behind the previous one made on another stream, so both streams finish with correct results."""
    m, n, k = 1024, 1536, 4096
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    data = []
    for seed in (51, 52):
        A, lda, B, ldb, C, ldc = make_dense("bf16", 0, 1, m, n, k, seed=seed, scale=0.25)
        data.append((A.to(DEV), B.to(DEV), torch.empty(m, n, dtype=torch.bfloat16, device=DEV), A, B))
    torch.cuda.synchronize()
    for _ in range(10):
        for s, (Ad, Bd, Cd, _, _) in zip((s1, s2), data):
            with torch.cuda.stream(s):
                fb.bfgemm(0, 1, m, n, k, 1.0, Ad, k, Bd, k, 0.0, Cd, n)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    for Ad, Bd, Cd, A, B in data:
        ref = (Ad.double() @ Bd.double().t()).float().cpu()
        assert_parity(Cd.float().cpu(), ref, KINDS["bf16"][2], result_scale(k, A, B, 1.0), "two streams")


@pytest.mark.parametrize("kind,ta,tb,m,n,k", [
    ("fp16", 0, 0, 8192, 1024, 8192),    # 128 tiles on 74 CTA pairs (one rank's share of 8192^3 over eight GPUs): 1.73 waves
    ("bf16", 0, 1, 2048, 4096, 2048),    # the same tile count, short k (16 stages), K-contiguous B
    ("tf32", 1, 0, 2304, 4096, 4096),    # 144 tiles: 1.95 waves, ranges that end a few stages into a tile
    ("bf16", 0, 0, 5000, 2500, 4096),    # 200 tiles = 2.7 waves with ragged edge tiles
])
def test_stream_k_over_the_last_wave(kind, ta, tb, m, n, k, monkeypatch):
    """Opt-in schedules for two or three waves of tiles of which the last is more than half full
    (FLAGBLAS_B200_STREAMK_FULL=1: whole waves first, then the k stages of the remaining tiles dealt evenly over all
    workers; =2: the stages of every tile dealt out): same results as whole tiles within the operator's tolerance."""
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=33, scale=0.25)
    Ad, Bd = A.to(DEV), B.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    outs = {}
    for mode in ("0", "1", "2"):
        monkeypatch.setenv("FLAGBLAS_B200_STREAMK_FULL", mode)
        fb.reload_env()
        Cd = C.to(DEV)
        op(ta, tb, m, n, k, 1.5, Ad, lda, Bd, ldb, 0.5, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        outs[mode] = Cd.float().cpu()
    sc = result_scale(k, A, B, 1.5) + 0.5
    opA = (Ad.t() if ta else Ad).double()
    opB = (Bd.t() if tb else Bd).double()
    if kind == "tf32":
        trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
        opA, opB = trunc(opA), trunc(opB)
    ref = (1.5 * (opA @ opB) + 0.5 * C.to(DEV).double()).float().cpu()
    for mode in ("0", "1", "2"):
        assert_parity(outs[mode], ref, KINDS[kind][2], sc, "last-wave stream-k=%s %s %dx%dx%d" % (mode, kind, m, n, k))


@pytest.mark.parametrize("kind,ta,tb,m,n,k", [
    ("fp16", 0, 0, 8192, 1024, 8192),    # one whole wave, then 54 tiles on 74 CTA pairs: 20 helpers, three tails each
    ("bf16", 0, 1, 2560, 1280, 8192),    # 50 tiles: no whole wave before the shared one
    ("tf32", 1, 0, 2048, 4096, 8192),    # 128 tiles, 256 k-slabs
    ("bf16", 0, 0, 5000, 1500, 8192),    # 120 tiles with ragged edge tiles: 28 helpers, two tails each
])
def test_tails_of_a_last_wave_go_to_idle_workers(kind, ta, tb, m, n, k, monkeypatch):
    """A last wave more than half full: the workers it would leave idle take the last k stages of its tiles
    (FLAGBLAS_B200_STREAMK_TAILS=0 keeps whole tiles).  Both plans agree with the fp64 product."""
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=35, scale=0.25)
    Ad, Bd = A.to(DEV), B.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    outs = {}
    monkeypatch.setenv("FLAGBLAS_B200_WIDE_TILES", "0")  # (a very long k would take one wave of 512-wide tiles instead)
    for mode in ("0", "1"):
        monkeypatch.setenv("FLAGBLAS_B200_STREAMK_TAILS", mode)
        fb.reload_env()
        Cd = C.to(DEV)
        op(ta, tb, m, n, k, 1.5, Ad, lda, Bd, ldb, 0.5, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        outs[mode] = Cd.float().cpu()
    sc = result_scale(k, A, B, 1.5) + 0.5
    opA = (Ad.t() if ta else Ad).double()
    opB = (Bd.t() if tb else Bd).double()
    if kind == "tf32":
        trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
        opA, opB = trunc(opA), trunc(opB)
    ref = (1.5 * (opA @ opB) + 0.5 * C.to(DEV).double()).float().cpu()
    for mode in ("0", "1"):
        assert_parity(outs[mode], ref, KINDS[kind][2], sc, "tails=%s %s %dx%dx%d" % (mode, kind, m, n, k))
    assert not torch.equal(outs["0"], outs["1"])  # another summation order somewhere: the second plan really ran


@pytest.mark.parametrize("kind,ta,tb,m,n,k", [
    ("fp16", 0, 0, 8192, 1024, 8192),    # 64 tiles of 256 x 512 on 74 CTA pairs (one rank's share of 8192^3 over eight GPUs)
    ("bf16", 0, 1, 4096, 2048, 4096),    # the same count, K-contiguous B
    ("tf32", 1, 0, 4096, 2048, 2048),    # TF32, A transposed
])
def test_single_wave_of_wide_tiles(kind, ta, tb, m, n, k, monkeypatch):
    """beta = 0 calls whose 512-wide tiles fill more than three quarters of one wave take them instead of two waves of
    256-wide tiles (FLAGBLAS_B200_WIDE_TILES=0 keeps the narrow ones): both agree with the fp64 product."""
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=37, scale=0.25)
    Ad, Bd = A.to(DEV), B.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    opA = (Ad.t() if ta else Ad).double()
    opB = (Bd.t() if tb else Bd).double()
    if kind == "tf32":
        trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
        opA, opB = trunc(opA), trunc(opB)
    ref = (1.5 * (opA @ opB)).float().cpu()
    sc = result_scale(k, A, B, 1.5)
    for mode in ("1", "0"):
        monkeypatch.setenv("FLAGBLAS_B200_WIDE_TILES", mode)
        fb.reload_env()
        Cd = torch.full((m, ldc), float("nan"), dtype=C.dtype, device=DEV)  # beta = 0 must not read C
        op(ta, tb, m, n, k, 1.5, Ad, lda, Bd, ldb, 0.0, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], sc, "wide=%s %s %dx%dx%d" % (mode, kind, m, n, k))


@pytest.mark.parametrize("kind,ta,tb,m,n,k,beta", [
    ("bf16", 0, 1, 16, 4096, 4096, 0.0),     # a few tokens against a square weight matrix, stored [n, k]
    ("bf16", 0, 0, 64, 2048, 8192, 0.5),     # stored [k, n], beta != 0
    ("fp16", 0, 1, 1, 4104, 4096, 0.0),      # one row, ragged n
    ("tf32", 1, 0, 33, 1000, 6144, 0.5),     # A transposed, n not a multiple of 4 (scalar stores of the parts)
    ("bf16", 0, 1, 128, 512, 16384, 0.0),    # very long k, four tiles
    ("bf16", 0, 1, 200, 200, 20000, 0.5),    # CTA-pair tile, one output tile, deep k
    ("fp16", 0, 0, 129, 2048, 4096, 0.0),    # CTA-pair tiles, eight output tiles
    ("tf32", 1, 1, 300, 520, 8192, 0.5),     # CTA-pair tiles, ragged
    ("bf16", 0, 1, 1024, 1024, 1024, 0.5),   # small square problem: 128-row tiles in clusters instead of CTA pairs
    ("bf16", 1, 0, 100, 264, 1024, 0.0),     # k barely long enough, ragged rows and columns
    ("tf32", 0, 1, 40, 520, 2048, 0.5),      # TF32 with k-contiguous A: five 8-row groups per A slot
    ("fp16", 0, 0, 7, 300, 512, 0.0),        # fewer rows than one 8-row group
    ("bf16", 0, 1, 119, 256, 4096, 0.5),     # the most rows that still shorten the A slots (120)
    ("bf16", 0, 1, 64, 6144, 2048, 0.0),     # 64 rows of 256-wide tiles: too large a tile to be sent, short A slots
    ("fp16", 0, 1, 96, 4096, 4096, 0.5),     # the same with 96 rows of 128-wide tiles
])
def test_split_k_for_skinny_shapes(kind, ta, tb, m, n, k, beta, monkeypatch):
    """Shapes with few output tiles and a long k are cut along k.  The parts are added either by the CTAs of a
    cluster over distributed shared memory (2, 4 or 8 parts; sent to the finishing CTA or read by it) or by a second
    kernel from fp32 scratch, and A's stage slots hold only as many rows as exist.  Same tolerance as every dense
    test; whole-k tiles, every forced cluster size in both forms, a forced part count of the scratch method and
    128-row A slots must agree with the automatic plan."""
    A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=41, scale=0.25)
    Ad, Bd = A.to(DEV), B.to(DEV)
    op = getattr(fb, KINDS[kind][1])
    opA = (Ad.t() if ta else Ad).double()
    opB = (Bd.t() if tb else Bd).double()
    if kind == "tf32":
        trunc = lambda x: (x.float().contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32).double()  # noqa: E731
        opA, opB = trunc(opA), trunc(opB)
    ref = (1.5 * (opA @ opB) + beta * C.to(DEV).double()).float().cpu()
    sc = result_scale(k, A, B, 1.5) + abs(beta)
    # switches of each mode (the others unset).  FLAGBLAS_B200_CLUSTER_PUSH=0: the finishing CTA reads its peers'
    # shared memory instead of being sent the sums; FLAGBLAS_B200_A_ROWS=0: 128-row A slots however few rows exist
    names = ("FLAGBLAS_B200_SPLITK", "FLAGBLAS_B200_CLUSTER_K", "FLAGBLAS_B200_PAIR", "FLAGBLAS_B200_CLUSTER_PUSH",
             "FLAGBLAS_B200_A_ROWS")
    cluster = lambda parts, **more: dict(FLAGBLAS_B200_SPLITK="0", FLAGBLAS_B200_CLUSTER_K=str(parts),  # noqa: E731
                                         FLAGBLAS_B200_PAIR="0", **more)
    modes = {"auto": {}, "whole-k": dict(FLAGBLAS_B200_SPLITK="0", FLAGBLAS_B200_CLUSTER_K="0"),
             "scratch-3": dict(FLAGBLAS_B200_SPLITK="3", FLAGBLAS_B200_CLUSTER_K="0"),
             "scratch-auto": dict(FLAGBLAS_B200_CLUSTER_K="0"),
             "cluster-2": cluster(2), "cluster-4": cluster(4), "cluster-8": cluster(8),
             "cluster-2-read": cluster(2, FLAGBLAS_B200_CLUSTER_PUSH="0"),
             "cluster-4-read": cluster(4, FLAGBLAS_B200_CLUSTER_PUSH="0", FLAGBLAS_B200_A_ROWS="0"),
             "cluster-8-read": cluster(8, FLAGBLAS_B200_CLUSTER_PUSH="0"),
             "cluster-2-sent-into-ring": cluster(2, FLAGBLAS_B200_CLUSTER_PUSH="2"),   # receiving area: the ring's end
             "cluster-4-sent-into-ring": cluster(4, FLAGBLAS_B200_CLUSTER_PUSH="2", FLAGBLAS_B200_A_ROWS="0"),
             "auto-whole-a-slots": dict(FLAGBLAS_B200_A_ROWS="0"),
             "cluster-4-whole-a-slots": cluster(4, FLAGBLAS_B200_A_ROWS="0")}
    for mode, envs in modes.items():
        for name in names:
            if name in envs:
                monkeypatch.setenv(name, envs[name])
            else:
                monkeypatch.delenv(name, raising=False)
        fb.reload_env()
        Cd = C.to(DEV) if beta != 0 else torch.full_like(C, float("nan")).to(DEV)
        op(ta, tb, m, n, k, 1.5, Ad, lda, Bd, ldb, beta, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], sc, "split-k %s %s %dx%dx%d" % (mode, kind, m, n, k))
    for name in names:
        monkeypatch.delenv(name, raising=False)
    monkeypatch.setenv("FLAGBLAS_B200_CLUSTER_K", "0")
    fb.reload_env()
    need = fb.c_operators.gemm_workspace_bytes(fb._lib.FB_BF16, 0, 1, 16, 4096, 4096, 256, 4096, 512, 4096)
    assert need >= 2 * 16 * 4096 * 4          # without clusters the first shape's plan asks for scratch for >= 2 parts


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp32"])
def test_one_row_or_column_goes_through_gemv(kind, monkeypatch):
    """m == 1 or n == 1: the call is a matrix-vector product and runs on the gemv kernels; same results (within the
    dense tolerance) as the tile kernels (FLAGBLAS_B200_GEMM_AS_GEMV=0), for every transposition and padded pitches."""
    op = getattr(fb, KINDS[kind][1])
    for (m, n, k) in [(1, 1000, 520), (700, 1, 264), (1, 1, 40)]:
        for ta in (0, 1):
            for tb in (0, 1):
                A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, pad=8, seed=51)
                ref = oracle_dense(kind, ta, tb, m, n, k, 1.5, A, lda, B, ldb, 0.5, C, ldc)
                for mode in ("1", "0"):
                    monkeypatch.setenv("FLAGBLAS_B200_GEMM_AS_GEMV", mode)
                    fb.reload_env()
                    Cd = C.to(DEV)
                    op(ta, tb, m, n, k, 1.5, A.to(DEV), lda, B.to(DEV), ldb, 0.5, Cd, ldc)
                    torch.cuda.synchronize()
                    assert fb.device_status() == 0
                    assert torch.equal(Cd.cpu()[:, n:], C[:, n:])
                    assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], result_scale(k, A, B, 1.5) + 0.5,
                                  "%s gemv=%s %dx%dx%d ta=%d tb=%d" % (kind, mode, m, n, k, ta, tb))
