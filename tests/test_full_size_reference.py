"""The benchmark workloads at full size against the reference's own output on the same seeded inputs.

``tests/golden/gpu_reference_full_size.npz`` (made by ``tests/golden/make_golden_gpu.py full_size`` on a B200) keeps whole
rows and whole columns of what the reference's generic Triton kernels computed for: fp16 8192^3, the bf16 MLP shape
(M = 16384, N = 14336, K = 4096, beta = 1), the 64-expert MoE, and the two TF32 contractions (16384^3 and the 64-row
skinny one; the reference has TF32 only as ``group_tf32gemm``, so those ran as one group).  The inputs are
regenerated from the seeds in ``gpu_cases``; a few input elements stored beside the outputs detect a generator
mismatch.  Tolerances are the operator's: rtol 1e-2 for fp16 / bf16, 1e-3 for TF32, plus the same rtol times the
typical output magnitude as the absolute term.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import gpu_cases as gc  # noqa: E402

from tests.helpers import KINDS, assert_parity  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def z(golden_dir):
    return np.load(os.path.join(golden_dir, "gpu_reference_full_size.npz"))


def _probe_ok(z, key, A, B):
    got = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
    np.testing.assert_array_equal(got, z[key + "_probe"], err_msg="input generator differs from the fixture's")


@pytest.mark.parametrize("name", list(gc.FULL_SIZE))
def test_dense_full_size_vs_reference_samples(z, name):
    import flagblas_b200 as fb

    kind, ta, tb, m, n, k, alpha, beta, A, B, C = gc.full_size_dense(name)
    _probe_ok(z, name, A, B)
    rms = lambda t: float(t[:64].float().pow(2).mean().sqrt())  # noqa: E731
    scale = abs(alpha) * k ** 0.5 * rms(A) * rms(B) + abs(beta) * rms(C)
    Ad, Bd = A.to(DEV), B.to(DEV)
    Cd = torch.full_like(C, float("nan")).to(DEV) if beta == 0.0 else C.to(DEV)
    getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, alpha, Ad, A.shape[1], Bd, B.shape[1], beta, Cd, n)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    rows, cols = [int(v) for v in z[name + "_rows"]], [int(v) for v in z[name + "_cols"]]
    ref_rows = gc.unpack(z[name + "_row_vals"], kind).float()
    ref_cols = gc.unpack(z[name + "_col_vals"], kind).float()
    assert not torch.isnan(ref_rows).any() and not torch.isnan(ref_cols).any()
    assert_parity(Cd[rows].float().cpu(), ref_rows, KINDS[kind][2], scale, name + " rows vs reference")
    assert_parity(Cd[:, cols].float().cpu(), ref_cols, KINDS[kind][2], scale, name + " columns vs reference")


def test_moe_full_size_vs_reference_samples(z):
    import flagblas_b200 as fb

    ms, K, N, A, B = gc.moe_case()
    _probe_ok(z, "moe", A, B)
    assert ms == [int(v) for v in z["moe_ms"]]
    E, T = len(ms), sum(ms)
    Ad, Bd = A.to(DEV), B.to(DEV)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=DEV)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    ap, bp, op, s = [], [], [], 0
    for g, mg in enumerate(ms):
        ap.append(Ad.data_ptr() + s * K * 2); op.append(out.data_ptr() + s * N * 2); bp.append(Bd.data_ptr() + g * K * N * 2)
        s += mg
    fb.group_bfgemm(out, i64(ap), i64(bp), i64(op), i64(op), i32(ms), i32([N] * E), i32([K] * E), i32([K] * E),
                    i32([N] * E), i32([N] * E), E, T, N, K, 1.0, 0.0)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert not torch.isnan(out).any()
    scale = K ** 0.5 * 0.02
    rows = [int(v) for v in z["moe_rows"]]
    assert_parity(out[rows].float().cpu(), gc.unpack(z["moe_row_vals"], "bf16").float(), 1e-2, scale, "moe rows vs reference")
    assert_parity(out[:, gc.MOE_COLS].float().cpu(), gc.unpack(z["moe_col_vals"], "bf16").float(), 1e-2, scale,
                  "moe columns vs reference")
