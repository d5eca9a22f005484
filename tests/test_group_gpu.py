"""Parity of the grouped CUDA path against the CPU oracle and the reference-made golden vectors."""
import os

import numpy as np
import pytest
import torch

import flagblas_b200 as fb
from oracle import gemm_oracle as go
from tests.helpers import KINDS, assert_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"
FN = {"bf16": "group_bfgemm", "fp16": "group_hgemm", "tf32": "group_tf32gemm"}


def _i64(v):
    return torch.tensor(v, dtype=torch.int64, device=DEV)


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _run_group(kind, ms, K, N, alpha, beta, seed=0, var_nk=False, use_small_m=False):
    """Mirror of the reference tests' set-up (tests/test_group_bfgemm.py:99-160): one A buffer of
    stacked rows, per-group B, raw device pointer / size arrays."""
    dt = KINDS[kind][0]
    nk = kind == "tf32"                      # group_tf32gemm stores B_g as [n, k]
    E = len(ms)
    g = torch.Generator().manual_seed(seed)
    ks = [K - 8 * (i % 3) for i in range(E)] if var_nk else [K] * E
    ns = [N - 8 * (i % 2) for i in range(E)] if var_nk else [N] * E
    A = torch.randn(sum(ms), K, generator=g).to(dt)
    Bs = [(torch.randn(ks[i], ns[i], generator=g) * K ** -0.5).to(dt) for i in range(E)]
    C = torch.randn(sum(ms), N, generator=g).to(dt)
    out = torch.full_like(C, float("nan"))
    Ad, Cd, outd = A.to(DEV), C.to(DEV), out.to(DEV)
    Bd = [(b.t().contiguous() if nk else b).to(DEV) for b in Bs]
    es = A.element_size()
    ap, bp, cp, op, s = [], [], [], [], 0
    for i, mg in enumerate(ms):
        ap.append(Ad.data_ptr() + s * K * es)
        cp.append(Cd.data_ptr() + s * N * es)
        op.append(outd.data_ptr() + s * N * es)
        bp.append(Bd[i].data_ptr())
        s += mg
    ldb = [ks[i] if nk else ns[i] for i in range(E)]
    ret = getattr(fb, FN[kind])(outd, _i64(ap), _i64(bp), _i64(cp), _i64(op), _i32(ms), _i32(ns), _i32(ks), _i32([K] * E),
                                _i32(ldb), _i32([N] * E), E, sum(ms), N, K, alpha, beta, use_small_m=use_small_m)
    assert ret is outd
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    a_list, b_list, c_list, s = [], [], [], 0
    for i, mg in enumerate(ms):
        a_list.append(A[s:s + mg, :ks[i]].float().numpy())
        b_list.append(Bs[i].float().numpy())
        c_list.append(C[s:s + mg, :ns[i]].float().numpy())
        s += mg
    refs = go.group_gemm(kind, a_list, b_list, c_list, alpha, beta, tf32_mode="trunc")
    got = outd.float().cpu()
    s = 0
    for i, mg in enumerate(ms):
        if mg:
            assert_parity(got[s:s + mg, :ns[i]], torch.from_numpy(refs[i]), KINDS[kind][2], abs(alpha) * 1.0 + abs(beta),
                          "%s group %d m=%d" % (kind, i, mg))
            if ns[i] < N:   # columns beyond n_g are never written
                assert torch.isnan(got[s:s + mg, ns[i]:]).all()
        s += mg
    return got


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_ragged(kind):
    _run_group(kind, [5, 0, 70, 33, 300, 128, 129, 1], 512, 384, 1.5, 0.5, seed=1)
    _run_group(kind, [128, 256], 256, 256, 1.0, 0.0, seed=2)
    _run_group(kind, [0, 0, 17], 64, 128, 1.0, 0.0, seed=3)
    _run_group(kind, [40, 200, 64], 200, 136, 1.5, 0.5, seed=4, var_nk=True)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_reference_shapes(kind):
    """A few of the reference's (k, e, n) grid (tests/accuracy_utils.py:299-330), m_g in [1, 512]."""
    import random
    rnd = random.Random(50)
    for (K, E, N) in [(64, 16, 128), (1024, 32, 512), (2048, 16, 1536)]:
        ms = [rnd.randint(1, 512) for _ in range(E)]
        _run_group(kind, ms, K, N, 1.5, 0.5, seed=K)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_alpha_zero_and_beta_zero(kind):
    got = _run_group(kind, [33, 64], 128, 128, 0.0, 0.5, seed=5)      # out = 0.5 * C
    assert not torch.isnan(got).any()
    got = _run_group(kind, [33, 64], 128, 128, 1.0, 0.0, seed=6)      # C pointers never dereferenced
    assert not torch.isnan(got).any()


@pytest.mark.parametrize("env", [{"FLAGBLAS_B200_GROUP_SPLIT": "1"}, {"FLAGBLAS_B200_GROUP_SPLIT": "2"}, {"FLAGBLAS_B200_PAIR": "0"},
                                 {"FLAGBLAS_B200_TMA3D": "0"},
                                 {"FLAGBLAS_B200_KS": "1"}, {"FLAGBLAS_B200_GROUP_SWAP": "0"},
                                 {"FLAGBLAS_B200_GROUP_SWAP": "0", "FLAGBLAS_B200_KS": "1"},
                                 {"FLAGBLAS_B200_GROUP_SMALL_M": "1"}, {"FLAGBLAS_B200_GROUP_SMALL_M": "1", "FLAGBLAS_B200_KS": "1"},
                                 {"FLAGBLAS_B200_GROUP_SMALL_M": "0"}])
def test_grouped_tile_plan_variants(env, monkeypatch):
    """The alternative tile plans (two-pass split of every remainder or only of remainders up to 128 rows,
    single-CTA tiles, 2-D copies, one k-slab per stage) compute the same thing."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
        fb.reload_env()
    _run_group("bf16", [5, 0, 70, 33, 300, 128, 129, 1, 700, 256], 512, 384, 1.5, 0.5, seed=11)
    _run_group("tf32", [40, 200, 64, 513], 200, 136, 1.5, 0.5, seed=12, var_nk=True)


@pytest.mark.parametrize("kind", ["bf16", "tf32"])
def test_grouped_stream_k_tail(kind, monkeypatch):
    """A grouped call whose last wave of tiles is at most half full shares each tail tile between 2-4 workers (the
    split is derived on the device).  Long k so that the split is worth it; FLAGBLAS_B200_GROUP_STREAMK=0 (whole
    tiles) must agree to the output type's rounding."""
    outs = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("FLAGBLAS_B200_GROUP_STREAMK", mode)
        fb.reload_env()
        outs[mode] = _run_group(kind, [300, 100, 0, 520, 77], 4096 if kind == "tf32" else 8192, 512, 1.5, 0.5, seed=21)
    assert_parity(outs["1"], outs["0"], KINDS[kind][2], 2.0, "grouped stream-k tail vs whole tiles")


def _run_group_general(kind, specs, alpha, beta, seed=0):
    """Grouped call in which every group has its own buffers, pitches and base offsets.
    spec = (m, n, k, lda_pad, ldb_pad, a_off, b_off): pads in elements on top of the tight pitch, offsets = elements
    by which the group's A / B start is shifted from its (256-byte aligned) allocation."""
    dt = KINDS[kind][0]
    nk = kind == "tf32"                      # group_tf32gemm stores B_g as [n, k]
    g = torch.Generator().manual_seed(seed)
    es = torch.empty(0, dtype=dt).element_size()
    keep, ptr, size, host = [], {c: [] for c in "abco"}, {c: [] for c in ("m", "n", "k", "lda", "ldb", "ldc")}, []
    for (m, n, k, lda_pad, ldb_pad, a_off, b_off) in specs:
        lda, ldb, ldc = k + lda_pad, (k if nk else n) + ldb_pad, n + 3
        A = torch.randn(m, lda, generator=g).to(dt)
        B = (torch.randn(n if nk else k, ldb, generator=g) * max(k, 1) ** -0.5).to(dt)
        C = torch.randn(m, ldc, generator=g).to(dt)
        bufs = []
        for t, off in ((A, a_off), (B, b_off), (C, 0), (torch.full_like(C, float("nan")), 0)):
            flat = torch.zeros(t.numel() + off + 64, dtype=dt, device=DEV)
            flat[off:off + t.numel()] = t.reshape(-1).to(DEV)
            bufs.append((flat, off))
        keep.append(bufs)
        for c, (flat, off) in zip("abco", bufs):
            ptr[c].append(flat.data_ptr() + off * es)
        for name, v in zip(("m", "n", "k", "lda", "ldb", "ldc"), (m, n, k, lda, ldb, ldc)):
            size[name].append(v)
        host.append((A, B, C))
    E = len(specs)
    outd = keep[0][3][0]
    getattr(fb, FN[kind])(outd, _i64(ptr["a"]), _i64(ptr["b"]), _i64(ptr["c"]), _i64(ptr["o"]), _i32(size["m"]), _i32(size["n"]),
                          _i32(size["k"]), _i32(size["lda"]), _i32(size["ldb"]), _i32(size["ldc"]), E, sum(size["m"]),
                          max(size["n"]), max(size["k"]), alpha, beta)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    for i, (m, n, k, *_rest) in enumerate(specs):
        if m == 0 or n == 0:
            continue
        A, B, C = host[i]
        a = A[:, :k].float().numpy()
        b = (B[:, :k].t() if nk else B[:, :n]).float().numpy()
        c = C[:, :n].float().numpy()
        ref = go.group_gemm(kind, [a], [b], [c], alpha, beta, tf32_mode="trunc")[0]
        flat, off = keep[i][3]
        got = flat[off:off + m * (n + 3)].reshape(m, n + 3).float().cpu()
        assert_parity(got[:, :n], torch.from_numpy(ref), KINDS[kind][2], abs(alpha) + abs(beta),
                      "%s general group %d (m=%d n=%d k=%d)" % (kind, i, m, n, k))
        assert torch.isnan(got[:, n:]).all(), "padding columns of the output were written"


# (m, n, k, lda_pad, ldb_pad, a_off, b_off)
_UNALIGNED_SPECS = [
    (70, 136, 100, 0, 0, 0, 0),      # k = 100: 16-bit rows of A are only 8-byte aligned
    (300, 200, 101, 0, 0, 0, 0),     # odd k: element-aligned rows of A (and of an [n, k] B)
    (129, 256, 256, 0, 0, 1, 1),     # aligned pitches, both bases shifted by one element
    (64, 128, 128, 0, 0, 0, 0),      # fully aligned group in the same call (stays on TMA)
    (260, 130, 192, 0, 1, 0, 0),     # odd ldb
    (0, 64, 64, 1, 1, 1, 1),         # empty group
    (33, 72, 40, 3, 5, 2, 3),        # everything odd, k shorter than a stage
    (513, 264, 520, 2, 0, 0, 0),     # several row tiles; A by hand, B by TMA
]


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_unaligned_operands(kind):
    """Groups whose A / B base or pitch is not 16-byte aligned (the reference takes any: block pointers with
    boundary checks, ops/level3/group_gemm.py:162-185) are computed by the producers' load / store path, mixed in
    one call with groups that stay on TMA."""
    _run_group_general(kind, _UNALIGNED_SPECS, 1.5, 0.5, seed=31)
    _run_group_general(kind, _UNALIGNED_SPECS[:3], 1.0, 0.0, seed=32)


@pytest.mark.parametrize("env", [{}, {"FLAGBLAS_B200_PAIR": "0"}, {"FLAGBLAS_B200_KS": "1"}, {"FLAGBLAS_B200_GROUP_SPLIT": "2"},
                                 {"FLAGBLAS_B200_GROUP_SWAP": "0"}, {"FLAGBLAS_B200_GROUP_SMALL_M": "1"}])
def test_grouped_by_hand_matches_tma(env, monkeypatch):
    """Every operand through the load / store path (FLAGBLAS_B200_GROUP_BY_HAND=1), aligned or not, in each tile plan:
    bit for bit what the TMA path gives."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    outs = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("FLAGBLAS_B200_GROUP_BY_HAND", mode)
        fb.reload_env()
        outs[mode] = [_run_group("bf16", [5, 0, 70, 33, 300, 128, 129, 1, 700, 256], 512, 384, 1.5, 0.5, seed=11),
                      _run_group("tf32", [40, 200, 64, 513], 200, 136, 1.5, 0.5, seed=12, var_nk=True),
                      _run_group("fp16", [100, 260], 1024, 128, 1.0, 0.0, seed=13)]
    for a, b in zip(outs["0"], outs["1"]):
        assert torch.equal(torch.nan_to_num(a, nan=-7.0), torch.nan_to_num(b, nan=-7.0))


def test_group_mm_unaligned_and_fp32(monkeypatch):
    """group_mm with pitches TMA cannot address, including fp32 (TF32 products) with B stored [k, n]: the by-hand
    producer then writes the 32-byte-atom swizzle of N-contiguous 32-bit operands."""
    g = torch.Generator().manual_seed(41)
    offs = torch.tensor([20, 20, 300, 433], dtype=torch.int32)
    for dt, kind, K, N in ((torch.float32, "tf32", 102, 66), (torch.float32, "tf32", 128, 136), (torch.bfloat16, "bf16", 100, 129),
                           (torch.float16, "fp16", 264, 320)):
        A = torch.randn(433, K, generator=g).to(dt)
        B = (torch.randn(4, K, N, generator=g) * K ** -0.5).to(dt)
        ref = torch.from_numpy(go.group_mm(kind, A.float().numpy(), B.float().numpy(), offs.numpy()))
        for mode in ("0", "1"):
            monkeypatch.setenv("FLAGBLAS_B200_GROUP_BY_HAND", mode)
            fb.reload_env()
            C = fb.group_mm(A.to(DEV), B.to(DEV), offs.to(DEV))
            torch.cuda.synchronize()
            assert fb.device_status() == 0
            assert_parity(C.float().cpu(), ref, KINDS[kind][2], 1.0, "group_mm %s K=%d N=%d by_hand=%s" % (kind, K, N, mode))


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_partial_blocks_every_row_count(kind):
    """A group's last, partial 256-row block is computed transposed with its row count (rounded up to 16) in the
    MMA's N slot: every residue class of the row count, alone and behind whole blocks, ragged n and k."""
    ms = [1, 15, 16, 17, 31, 32, 33, 64, 100, 127, 128, 129, 200, 240, 241, 255, 256, 257, 256 + 16, 512 + 250, 0, 3 * 256]
    _run_group(kind, ms, 256, 520, 1.5, 0.5, seed=51)
    _run_group(kind, ms[:12], 200, 136, 1.0, 0.0, seed=52, var_nk=True)


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
def test_grouped_decode_shape_small_m(kind, monkeypatch):
    """The reference's small-M case (every m_g <= 64, use_small_m=True routes to its dedicated kernels,
    runtime/backend/_nvidia/hopper/ops/group_gemm.py:717-721): here the small-M plan -- every tile a transposed block of
    up to 64 rows, 32-row A slots, a deeper ring.  The promise is not relied on: groups with more rows are tiled in
    64-row blocks.  Same bits as the general plan."""
    import random
    rnd = random.Random(7)
    ms = [rnd.randint(0, 64) for _ in range(64)]
    got = _run_group(kind, ms, 1024, 768, 1.5, 0.5, seed=53, use_small_m=True)
    monkeypatch.setenv("FLAGBLAS_B200_GROUP_SMALL_M", "0")
    fb.reload_env()
    ref = _run_group(kind, ms, 1024, 768, 1.5, 0.5, seed=53, use_small_m=True)
    assert torch.equal(torch.nan_to_num(got, nan=-7.0), torch.nan_to_num(ref, nan=-7.0))
    monkeypatch.delenv("FLAGBLAS_B200_GROUP_SMALL_M")
    fb.reload_env()
    # the promise broken: a 700-row and a 65-row group among the small ones
    _run_group(kind, [3, 700, 64, 65, 0, 17, 129], 520, 264, 1.5, 0.5, seed=54, use_small_m=True)
    _run_group(kind, [40, 200, 64, 33], 200, 136, 1.0, 0.0, seed=55, var_nk=True, use_small_m=True)


def test_group_prepare_then_run_matches_the_plain_call():
    """Tables and tensor maps built once (fb_group_gemm_prepare), the GEMM run several times over them
    (fb_group_gemm_run) with different scalars and new operand data: bit for bit what the plain call gives."""
    g = torch.Generator().manual_seed(61)
    ms, K, N = [300, 0, 70, 512, 33, 1], 512, 384
    E, T = len(ms), sum(ms)
    A = torch.randn(T, K, generator=g).bfloat16().to(DEV)
    B = (torch.randn(E * K, N, generator=g) * K ** -0.5).bfloat16().to(DEV)
    C = torch.randn(T, N, generator=g).bfloat16().to(DEV)
    starts = [sum(ms[:e]) for e in range(E)]

    def arrays(out):
        return (_i64([A.data_ptr() + s * K * 2 for s in starts]), _i64([B.data_ptr() + e * K * N * 2 for e in range(E)]),
                _i64([C.data_ptr() + s * N * 2 for s in starts]), _i64([out.data_ptr() + s * N * 2 for s in starts]),
                _i32(ms), _i32([N] * E), _i32([K] * E), _i32([K] * E), _i32([N] * E), _i32([N] * E))

    out_p = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    plan = fb.group_prepare("group_bfgemm", *arrays(out_p), E, T, N, K)
    for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
        out_ref = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        fb.group_bfgemm(out_ref, *arrays(out_ref), E, T, N, K, alpha, beta)
        assert plan.run(out_p, alpha, beta) is out_p
        torch.cuda.synchronize()
        assert torch.equal(out_p, out_ref)
        A.mul_(0.5)          # new data in the same buffers: the plan holds addresses, not values
    assert not torch.isnan(out_p).any()
    assert fb.device_status() == 0


def test_grouped_many_groups():
    _run_group("bf16", [((7 * i) % 90) for i in range(600)], 128, 256, 1.0, 0.0, seed=7)
    # more groups than the table builder keeps in shared memory (its tile counts then go through global memory)
    _run_group("fp16", [((5 * i) % 23) for i in range(1500)], 64, 128, 1.0, 0.0, seed=8)


def test_group_mm_and_group_gemm():
    g = torch.Generator().manual_seed(8)
    for dt, kind in ((torch.float16, "fp16"), (torch.bfloat16, "bf16")):
        A = torch.randn(432, 256, generator=g).to(dt)
        B = (torch.randn(4, 256, 320, generator=g) / 16).to(dt)
        offs = torch.tensor([20, 20, 300, 432], dtype=torch.int32)
        C = fb.group_mm(A.to(DEV), B.to(DEV), offs.to(DEV))
        ref = go.group_mm(kind, A.float().numpy(), B.float().numpy(), offs.numpy())
        assert_parity(C.float().cpu(), torch.from_numpy(ref), 1e-2, 1.0, "group_mm " + kind)
        # B given as a transposed view ([G, N, K] storage)
        Bt = B.transpose(1, 2).contiguous().transpose(1, 2)
        C2 = fb.group_mm(A.to(DEV), Bt.to(DEV), offs.to(DEV))
        assert_parity(C2.float().cpu(), torch.from_numpy(ref), 1e-2, 1.0, "group_mm K-contiguous B " + kind)
        # group_gemm: offs_table rows = [m, n, k, start_M, start_K, start_C]
        ms = [20, 0, 280, 132]
        table, s = [], 0
        for i, mg in enumerate(ms):
            table.append([mg, 320, 256, s, i * 256, s])
            s += mg
        Cin = torch.randn(432, 320, generator=g).to(dt)
        out = fb.group_gemm(A.to(DEV), B.reshape(4 * 256, 320).to(DEV), Cin.to(DEV), table, alpha=1.5, beta=0.5)
        a_list, c_list, s = [], [], 0
        for mg in ms:
            a_list.append(A[s:s + mg].float().numpy()); c_list.append(Cin[s:s + mg].float().numpy()); s += mg
        refs = go.group_gemm(kind, a_list, [B[i].float().numpy() for i in range(4)], c_list, 1.5, 0.5)
        assert_parity(out.float().cpu(), torch.from_numpy(np.concatenate(refs, 0)), 1e-2, 2.0, "group_gemm " + kind)


def test_group_gemm_fp32_runs_tf32():
    """group_gemm on fp32 tensors: TF32 products with B_g stored [k, n] (not a 16-bit kernel over fp32 storage)."""
    g = torch.Generator().manual_seed(9)
    ms, K, N = [20, 0, 280, 132], 256, 320
    A = torch.randn(sum(ms), K, generator=g)
    B = torch.randn(4 * K, N, generator=g) / 16
    Cin = torch.randn(sum(ms), N, generator=g)
    table, s = [], 0
    for i, mg in enumerate(ms):
        table.append([mg, N, K, s, i * K, s])
        s += mg
    out = fb.group_gemm(A.to(DEV), B.to(DEV), Cin.to(DEV), table, alpha=1.5, beta=0.5)
    a_list, c_list, s = [], [], 0
    for mg in ms:
        a_list.append(A[s:s + mg].numpy()); c_list.append(Cin[s:s + mg].numpy()); s += mg
    refs = go.group_gemm("tf32", a_list, [B[i * K:(i + 1) * K].numpy() for i in range(4)], c_list, 1.5, 0.5)
    assert_parity(out.float().cpu(), torch.from_numpy(np.concatenate(refs, 0)), 1e-3, 2.0, "group_gemm fp32")
    assert fb.device_status() == 0


def test_golden_grouped_on_gpu(golden_dir):
    z = np.load(os.path.join(golden_dir, "grouped.npz"))
    for name, kind in (("h", "fp16"), ("tf32", "tf32")):
        for tag in ("ab", "b0"):
            pre = "g%s_%s_" % (name, tag)
            p = z[pre + "p"]
            ms = [int(v) for v in p[:4]]
            K, N, al, be = int(p[4]), int(p[5]), float(p[6]), float(p[7])
            dt = KINDS[kind][0]
            nk = kind == "tf32"
            A = torch.from_numpy(z[pre + "A"]).to(dt).to(DEV)
            B = torch.from_numpy(z[pre + "B"]).to(dt)
            Bd = [(B[i * K:(i + 1) * K].t().contiguous() if nk else B[i * K:(i + 1) * K].contiguous()).to(DEV) for i in range(4)]
            C = torch.from_numpy(z[pre + "C"]).to(dt).to(DEV)
            out = torch.full_like(C, float("nan"))
            es = A.element_size()
            ap, cp, op, s = [], [], [], 0
            for mg in ms:
                ap.append(A.data_ptr() + s * K * es); cp.append(C.data_ptr() + s * N * es); op.append(out.data_ptr() + s * N * es); s += mg
            getattr(fb, FN[kind])(out, _i64(ap), _i64([b.data_ptr() for b in Bd]), _i64(cp), _i64(op), _i32(ms), _i32([N] * 4),
                                  _i32([K] * 4), _i32([K] * 4), _i32([K if nk else N] * 4), _i32([N] * 4), 4, sum(ms), N, K, al, be)
            ref = torch.from_numpy(z[pre + "out"])
            # the tf32 golden vectors were computed in full fp32 (Triton's CPU interpreter does not
            # round to TF32) while the tensor core truncates the inputs: allow 4x the typical size
            sc = (abs(al) + abs(be)) * (4.0 if kind == "tf32" else 1.0)
            assert_parity(out.float().cpu(), ref, KINDS[kind][2], sc, "golden " + pre)
    A = torch.from_numpy(z["mm_A"]).half().to(DEV)
    B = torch.from_numpy(z["mm_B"]).half().to(DEV)
    C = fb.group_mm(A, B, torch.from_numpy(z["mm_offs"]).to(DEV))
    assert_parity(C.float().cpu()[:108], torch.from_numpy(z["mm_C"])[:108], 1e-2, 8.0, "golden group_mm")


def test_moe_config4_properties():
    """The grouped MoE benchmark workload at full size: 64 experts, K=4096, N=1536, Zipf(1.2) token counts (zeros allowed)."""
    E, K, N, T = 64, 4096, 1536, 32768
    g = torch.Generator().manual_seed(3)
    w = torch.arange(1, E + 1, dtype=torch.float64) ** -1.2
    ms = torch.multinomial(w / w.sum(), T, replacement=True, generator=g).bincount(minlength=E).tolist()
    gd = torch.Generator(device=DEV).manual_seed(3)
    A = torch.randn(T, K, generator=gd, device=DEV).bfloat16()
    B = (torch.randn(E * K, N, generator=gd, device=DEV) * 0.02).bfloat16()
    out = torch.full((T, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    ap, bp, op, s = [], [], [], 0
    for i, mg in enumerate(ms):
        ap.append(A.data_ptr() + s * K * 2); bp.append(B.data_ptr() + i * K * N * 2); op.append(out.data_ptr() + s * N * 2); s += mg
    fb.group_bfgemm(out, _i64(ap), _i64(bp), _i64(op), _i64(op), _i32(ms), _i32([N] * E), _i32([K] * E), _i32([K] * E),
                    _i32([N] * E), _i32([N] * E), E, T, N, K, 1.0, 0.0)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert not torch.isnan(out).any()
    sc = (K ** 0.5) * 0.02
    s = 0
    for i, mg in enumerate(ms):
        if mg:
            rows = sorted({s, s + mg // 2, s + mg - 1})
            ref = A[rows].double() @ B[i * K:(i + 1) * K].double()
            assert_parity(out[rows].float().cpu(), ref.float().cpu(), 1e-2, sc, "moe expert %d" % i)
        s += mg


def test_bounded_wait_reports_timeout():
    """A wait on a barrier nothing completes gives up after its limit and reports it; the
    context stays usable afterwards."""
    assert fb.c_operators.selftest_bounded_wait(20_000_000, 0) == 105
    assert fb.device_status() == 0
    x = torch.ones(8, device=DEV)
    assert float(x.sum()) == 8.0


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_grouped_pieces_reassemble(world):
    """The multi-GPU grouped path on one GPU: every rank's pieces (row slices of groups, planned by
    FLOPs) run one after the other into one output must give, bit for bit, what a single call gives."""
    from flagblas_b200 import dist

    g = torch.Generator(device="cpu").manual_seed(9)
    ms, K, N = [700, 0, 130, 1100, 64, 257], 256, 384
    E, T = len(ms), sum(ms)
    A = torch.randn(T, K, generator=g).bfloat16().to(DEV)
    B = (torch.randn(E * K, N, generator=g) * K ** -0.5).bfloat16().to(DEV)
    starts = [sum(ms[:e]) for e in range(E)]
    a = [A.data_ptr() + s * K * 2 for s in starts]
    b = [B.data_ptr() + e * K * N * 2 for e in range(E)]

    def run(plan):
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        o = [out.data_ptr() + s * N * 2 for s in starts]
        for pieces in plan:
            arrays, cnt = dist.shard_group_arrays(pieces, a, b, o, o, ms, [N] * E, [K] * E, [K] * E, [N] * E, [N] * E,
                                                  2, DEV)
            if cnt:
                fb.group_bfgemm(out, *arrays, cnt, sum(r for _, _, r in pieces), N, K, 1.0, 0.0)
        torch.cuda.synchronize()
        return out

    whole = run(dist.plan_group_shards(ms, [N] * E, [K] * E, 1))
    parts = run(dist.plan_group_shards(ms, [N] * E, [K] * E, world, row_align=256))
    assert fb.device_status() == 0
    assert not torch.isnan(whole).any()
    assert torch.equal(whole, parts)
