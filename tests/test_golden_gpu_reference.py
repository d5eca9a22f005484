"""Golden vectors made by the reference's own Triton kernels running natively on a B200
(tests/golden/make_golden_gpu.py).  They pin what the CPU-interpreter vectors cannot: bfloat16
results, and the TF32 rounding of the reference's lowering -- which on B200 TRUNCATES the fp32
operands, exactly what tcgen05 does to raw fp32 words in shared memory.

CPU part: the oracle against these vectors.  GPU part: our kernels against them.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import gpu_cases as gc  # noqa: E402

from oracle import gemm_oracle as go  # noqa: E402
from tests.helpers import KINDS, assert_parity, result_scale  # noqa: E402


@pytest.fixture(scope="module")
def z(golden_dir):
    return np.load(os.path.join(golden_dir, "gpu_reference.npz"))


def _probe_ok(z, key, A, B):
    got = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
    np.testing.assert_array_equal(got, z[key + "_probe"], err_msg="input generator differs from the fixture's")


# ------------------------------------------------------------------------------------- oracle (CPU)
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp32"])
def test_oracle_dense_vs_reference_on_gpu(z, kind):
    for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.dense_cases(kind):
        _probe_ok(z, key, A, B)
        ref = gc.unpack(z[key + "_C"], kind).float().numpy()
        c = C.float().numpy().copy()
        go.gemm(kind, ta, tb, m, n, k, alpha, A.float().numpy(), lda, B.float().numpy(), ldb, beta, c, ldc)
        np.testing.assert_array_equal(ref[:, n:], C.float().numpy()[:, n:])   # reference leaves padding alone
        if kind == "fp32":
            np.testing.assert_allclose(c[:, :n], ref[:, :n], rtol=1e-5, atol=1e-5 * result_scale(k, A, B, alpha))
        else:
            # one rounding at the end on both sides: the same bits except where the fp32 sums straddle
            # a rounding boundary (then one unit in the last place apart)
            assert np.mean(c[:, :n] == ref[:, :n]) > 0.995, key
            ulp = 2.0 ** -7 if kind == "bf16" else 2.0 ** -10
            assert np.all(np.abs(c[:, :n] - ref[:, :n]) <= ulp * np.maximum(np.abs(ref[:, :n]), 1e-3) * 1.01), key


def _group_lists(kind, ms, K, A, B, C):
    a_list, b_list, c_list, s = [], [], [], 0
    for g, mg in enumerate(ms):
        a_list.append(A[s:s + mg].float().numpy())
        b_list.append(B[g * K:(g + 1) * K].float().numpy())
        c_list.append(C[s:s + mg].float().numpy())
        s += mg
    return a_list, b_list, c_list


@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
@pytest.mark.parametrize("tag", ["ab", "b0"])
def test_oracle_grouped_vs_reference_on_gpu(z, kind, tag):
    ms, K, N, al, be, A, B, C = gc.group_case(kind, tag)
    _probe_ok(z, "group_%s_%s" % (kind, tag), A, B)
    ref = gc.unpack(z["group_%s_%s_out" % (kind, tag)], kind).float().numpy()
    assert not np.isnan(ref).any()
    a_list, b_list, c_list = _group_lists(kind, ms, K, A, B, C)
    got = np.concatenate(go.group_gemm(kind, a_list, b_list, c_list, al, be, tf32_mode="trunc"), 0)
    if kind == "tf32":
        np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-5)       # truncating oracle: fp32-level agreement
        rna = np.concatenate(go.group_gemm(kind, a_list, b_list, c_list, al, be, tf32_mode="rna"), 0)
        assert np.abs(rna - ref).max() > 50 * np.abs(got - ref).max()    # ...and clearly not round-to-nearest
    else:
        assert np.mean(got == ref) > 0.995


def test_reference_truncates_tf32_on_b200(z):
    m, n, k, A, Bt = gc.tf32_probe()
    out = z["tf32probe_out"].astype(np.float64)
    a, b = A.numpy(), Bt.numpy()
    rel = {}
    for name, f in (("trunc", go.trunc_tf32), ("rna", go.round_tf32)):
        r = f(a).astype(np.float64) @ f(b).astype(np.float64).T
        rel[name] = float(np.mean((out - r) / r))
    assert abs(rel["trunc"]) < 5e-5 and rel["rna"] < -5e-4, rel


def test_oracle_group_mm_vs_reference_on_gpu(z):
    A, B, offs = gc.group_mm_case()
    ref = gc.unpack(z["mm_C"], "bf16").float().numpy()
    got = go.group_mm("bf16", A.float().numpy(), B.float().numpy(), offs.numpy())
    assert np.mean(got == ref) > 0.995


# ------------------------------------------------------------------------------------- our kernels (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp32"])
def test_kernels_dense_vs_reference_on_gpu(z, kind):
    import flagblas_b200 as fb

    for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.dense_cases(kind):
        ref = gc.unpack(z[key + "_C"], kind).float()
        Cd = C.to("cuda")
        getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, alpha, A.to("cuda"), lda, B.to("cuda"), ldb, beta, Cd, ldc)
        got = Cd.float().cpu()
        assert torch.equal(got[:, n:], ref[:, n:])
        assert_parity(got[:, :n], ref[:, :n], KINDS[kind][2], result_scale(k, A, B, alpha) + abs(beta), "vs reference on GPU " + key)
        if kind != "fp32":
            assert float((got[:, :n] == ref[:, :n]).float().mean()) > 0.99, key


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["bf16", "fp16", "tf32"])
@pytest.mark.parametrize("tag", ["ab", "b0"])
def test_kernels_grouped_vs_reference_on_gpu(z, kind, tag):
    import flagblas_b200 as fb

    dev = "cuda"
    ms, K, N, al, be, A, B, C = gc.group_case(kind, tag)
    E = len(ms)
    nk = kind == "tf32"
    ref = gc.unpack(z["group_%s_%s_out" % (kind, tag)], kind).float()
    Ad, Cd = A.to(dev), C.to(dev)
    Bd = (torch.cat([B[g * K:(g + 1) * K].t().contiguous() for g in range(E)], 0) if nk else B).to(dev)
    out = torch.full_like(Cd, float("nan"))
    es = A.element_size()
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    ap, bp, cp, op, s = [], [], [], [], 0
    for g, mg in enumerate(ms):
        ap.append(Ad.data_ptr() + s * K * es); cp.append(Cd.data_ptr() + s * N * es)
        op.append(out.data_ptr() + s * N * es); bp.append(Bd.data_ptr() + g * K * N * es)
        s += mg
    fn = {"bf16": fb.group_bfgemm, "fp16": fb.group_hgemm, "tf32": fb.group_tf32gemm}[kind]
    fn(out, i64(ap), i64(bp), i64(cp), i64(op), i32(ms), i32([N] * E), i32([K] * E), i32([K] * E), i32([K if nk else N] * E),
       i32([N] * E), E, sum(ms), N, K, al, be)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    got = out.float().cpu()
    # tf32: the reference truncates like the tensor core does, so the plain 1e-3 bound holds
    assert_parity(got, ref, KINDS[kind][2], abs(al) + abs(be), "grouped vs reference on GPU %s %s" % (kind, tag))
    if kind == "tf32":
        assert float((got - ref).abs().max()) < 5e-5


@pytest.mark.gpu
def test_kernels_tf32_probe_and_group_mm_vs_reference_on_gpu(z):
    import flagblas_b200 as fb

    m, n, k, A, Bt = gc.tf32_probe()
    ref = torch.from_numpy(z["tf32probe_out"])
    # dense tf32gemm with B stored [n, k] (transb = T) computes the same contraction
    C = torch.zeros(m, n, device="cuda")
    fb.tf32gemm(0, 1, m, n, k, 1.0, A.to("cuda"), k, Bt.to("cuda"), k, 0.0, C, n)
    rel = ((C.cpu().double() - ref.double()) / ref.double())
    assert float(rel.abs().max()) < 5e-5          # same truncation as the reference: fp32-level agreement
    A2, B2, offs = gc.group_mm_case()
    got = fb.group_mm(A2.to("cuda"), B2.to("cuda"), offs.to("cuda")).float().cpu()
    refmm = gc.unpack(z["mm_C"], "bf16").float()
    assert float((got[:216] == refmm[:216]).float().mean()) > 0.99
