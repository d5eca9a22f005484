"""The allocation-free grouped GEMM entry point (fb_group_gemm_no_alloc).

Some users of this library may not allocate device memory when they call it: plug-ins that run
inside another runtime's enqueue hook, and services that gave all of HBM to their own pool at
start-up.  For them the library keeps the grouped GEMM's scratch in a fixed built-in array.  This
test drives that entry point through the C ABI, twice in a row (the array is reused and keeps
whatever the previous call left in it), and requires the same bits as the ordinary entry point
that takes a caller-provided workspace.  It also checks the capacity limit is enforced.

Collected last on purpose (file name), so that a run stopping at the first failure has
already exercised everything else.
"""
import pytest
import torch

import flagblas_b200 as fb
from flagblas_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _problem(ms, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    E = len(ms)
    A = torch.randn(sum(ms), K, generator=g).bfloat16().to(DEV)
    B = (torch.randn(E, K, N, generator=g) / K ** 0.5).bfloat16().to(DEV)
    C = torch.randn(sum(ms), N, generator=g).bfloat16().to(DEV)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=DEV)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    ap, cp, s = [], [], 0
    for mg in ms:
        ap.append(A.data_ptr() + s * K * 2)
        cp.append(C.data_ptr() + s * N * 2)
        s += mg
    bp = [B.data_ptr() + e * K * N * 2 for e in range(E)]
    sizes = (i32(ms), i32([N] * E), i32([K] * E), i32([K] * E), i32([N] * E), i32([N] * E))
    return A, B, C, i64(ap), i64(bp), i64(cp), sizes, E


def _out_ptrs(out, ms, N):
    ptrs, s = [], 0
    for mg in ms:
        ptrs.append(out.data_ptr() + s * N * 2)
        s += mg
    return torch.tensor(ptrs, dtype=torch.int64, device=DEV)


def test_no_alloc_matches_workspace_entry_point_twice():
    L = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second one finds the first one's table in the array
    for ms, K, N, alpha, beta, seed in (([70, 0, 300, 5, 129], 512, 384, 1.5, 0.5, 1), ([256, 33], 256, 640, 1.0, 0.0, 2)):
        A, B, C, ap, bp, cp, sizes, E = _problem(ms, K, N, seed)
        ref = torch.full_like(C, float("nan"))
        got = torch.full_like(C, float("nan"))
        nbytes = L.fb_group_workspace_bytes(E)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        rc = L.fb_group_gemm(_lib.FB_BF16, 0, ap.data_ptr(), bp.data_ptr(), cp.data_ptr(), _out_ptrs(ref, ms, N).data_ptr(),
                             *[t.data_ptr() for t in sizes], E, sum(ms), N, K, alpha, beta, ws.data_ptr(), nbytes, stream)
        assert rc == 0
        rc = L.fb_group_gemm_no_alloc(_lib.FB_BF16, 0, ap.data_ptr(), bp.data_ptr(), cp.data_ptr(),
                                      _out_ptrs(got, ms, N).data_ptr(), *[t.data_ptr() for t in sizes], E, sum(ms), N, K,
                                      alpha, beta, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert not torch.isnan(got).any()
        assert torch.equal(got, ref)  # same kernels, same arithmetic: identical bits (tolerance 0)


def test_no_alloc_long_k_agrees_with_both_workspace_sizes():
    """Long k and few tiles: given its optional partial-sum scratch, the ordinary entry point shares each tile of the
    half-empty last wave between several CTAs (another summation order); the built-in array holds only the tables, so
    the allocation-free entry point runs whole tiles.  Its result is bit for bit that of the ordinary entry point with
    a tables-only workspace, and within the operator's tolerance of the one with the full workspace."""
    from tests.helpers import assert_parity

    L = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    ms, K, N, alpha, beta = [600, 100, 256], 8192, 512, 1.5, 0.5
    A, B, C, ap, bp, cp, sizes, E = _problem(ms, K, N, 3)
    outs = {}
    for name, nbytes in (("full", L.fb_group_workspace_bytes(E)), ("tables", L.fb_group_min_workspace_bytes(E))):
        assert nbytes > 0
        out = torch.full_like(C, float("nan"))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        rc = L.fb_group_gemm(_lib.FB_BF16, 0, ap.data_ptr(), bp.data_ptr(), cp.data_ptr(), _out_ptrs(out, ms, N).data_ptr(),
                             *[t.data_ptr() for t in sizes], E, sum(ms), N, K, alpha, beta, ws.data_ptr(), nbytes, stream)
        assert rc == 0
        torch.cuda.synchronize()
        outs[name] = out
    assert L.fb_group_workspace_bytes(E) > L.fb_group_min_workspace_bytes(E)
    for _ in range(2):
        got = torch.full_like(C, float("nan"))
        rc = L.fb_group_gemm_no_alloc(_lib.FB_BF16, 0, ap.data_ptr(), bp.data_ptr(), cp.data_ptr(),
                                      _out_ptrs(got, ms, N).data_ptr(), *[t.data_ptr() for t in sizes], E, sum(ms), N, K,
                                      alpha, beta, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert not torch.isnan(got).any()
        assert torch.equal(got, outs["tables"])
        assert_parity(got.float().cpu(), outs["full"].float().cpu(), 1e-2, abs(alpha) + abs(beta), "no-alloc vs full workspace")


def test_no_alloc_rejects_more_groups_than_it_can_hold():
    L = _lib.lib
    cap = L.fb_no_alloc_max_groups()
    assert cap == 256
    dummy = torch.zeros(8, dtype=torch.int64, device=DEV).data_ptr()
    rc = L.fb_group_gemm_no_alloc(_lib.FB_BF16, 0, *([dummy] * 10), cap + 1, 0, 0, 0, 1.0, 0.0, None)
    assert rc == -6
    assert b"capacity" in L.fb_status_string(rc)
