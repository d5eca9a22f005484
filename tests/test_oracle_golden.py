"""The CPU oracle against golden vectors made by the reference's own kernels
(tests/golden/make_golden.py).  Runs without a GPU."""
import os

import numpy as np
import pytest

from oracle import gemm_oracle as go


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("kind,rtol,atol", [("fp32", 2e-6, 2e-5), ("fp16", 1e-3, 1e-3)])
def test_dense_matches_reference(golden_dir, kind, rtol, atol):
    z = _load(golden_dir, "dense_%s.npz" % kind)
    keys = sorted(k[:-2] for k in z.files if k.endswith("_p"))
    assert len(keys) == 8
    for key in keys:
        ta, tb, m, n, k, lda, ldb, ldc, alpha, beta = z[key + "_p"]
        ta, tb, m, n, k, lda, ldb, ldc = (int(v) for v in (ta, tb, m, n, k, lda, ldb, ldc))
        c = z[key + "_C0"].copy()
        go.gemm(kind, ta, tb, m, n, k, alpha, z[key + "_A"], lda, z[key + "_B"], ldb, beta, c, ldc)
        ref = z[key + "_C"]
        # padding columns (ld > n) must be untouched by both
        np.testing.assert_array_equal(c[:, n:], z[key + "_C0"][:, n:])
        np.testing.assert_array_equal(ref[:, n:], z[key + "_C0"][:, n:])
        np.testing.assert_allclose(c[:, :n], ref[:, :n], rtol=rtol, atol=atol, err_msg=key)
        if kind == "fp16":
            # one rounding at the end: at most 1 fp16 ulp apart, and identical almost everywhere
            same = np.mean(c[:, :n] == ref[:, :n])
            assert same > 0.98, (key, same)


def test_edge_cases_match_reference(golden_dir):
    z = _load(golden_dir, "edge_fp32.npz")
    A, B, C0 = z["A"], z["B"], z["C0"]
    c = C0.copy(); go.gemm("fp32", 0, 0, 64, 64, 64, 0.0, A, 64, B, 64, 0.5, c, 64)
    np.testing.assert_array_equal(c, z["alpha_zero"])
    c = np.full_like(C0, np.nan); go.gemm("fp32", 0, 0, 64, 64, 64, 2.5, A, 64, B, 64, 0.0, c, 64)
    assert not np.isnan(z["beta_zero_nanC"]).any() and not np.isnan(c).any()
    np.testing.assert_allclose(c, z["beta_zero_nanC"], rtol=2e-6, atol=2e-5)
    c = C0[:1].copy(); go.gemm("fp32", 0, 0, 0, 64, 64, 2.5, A, 64, B, 64, 0.5, c, 64)
    np.testing.assert_array_equal(c, z["empty_m0"])          # whole (1 x 64) buffer halved
    c = C0.copy(); go.gemm("fp32", 0, 0, 64, 64, 0, 2.5, A, 64, B, 64, 0.5, c, 64)
    np.testing.assert_array_equal(c, z["empty_k0"])
    c = C0.copy(); go.gemm("fp32", 0, 0, 64, 0, 64, 2.5, A, 64, B, 64, 0.0, c, 64)
    np.testing.assert_array_equal(c, z["empty_n0_beta0"])
    for i in range(5):
        al, be = z["ab%d_p" % i]
        c = C0.copy(); go.gemm("fp32", 0, 0, 64, 64, 64, al, A, 64, B, 64, be, c, 64)
        np.testing.assert_allclose(c, z["ab%d" % i], rtol=2e-6, atol=2e-5)


def test_config1_sgemm512(golden_dir):
    """The small fp32 benchmark workload (sgemm 512^3, U(-1,1), seed 0) as the reference computed it on CPU."""
    import torch

    z = _load(golden_dir, "config1_sgemm512.npz")
    g = torch.Generator(device="cpu").manual_seed(0)
    A = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    B = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    np.testing.assert_array_equal(A[:4, :8], z["A_probe"])   # same generator stream as the fixture
    np.testing.assert_array_equal(B[:4, :8], z["B_probe"])
    C = np.zeros((512, 512), dtype=np.float32)
    go.gemm("fp32", 0, 0, 512, 512, 512, 1.0, A, 512, B, 512, 0.0, C, 512)
    np.testing.assert_allclose(C[::4, ::4], z["C_sub"], rtol=1e-5, atol=1e-5 * 13.0)
    assert abs(C.astype(np.float64).sum() - float(z["C_sum"])) < 1e-2


def test_grouped_matches_reference(golden_dir):
    z = _load(golden_dir, "grouped.npz")
    for name, kind, nk in (("h", "fp16", False), ("tf32", "tf32", True)):
        for tag in ("ab", "b0"):
            pre = "g%s_%s_" % (name, tag)
            p = z[pre + "p"]
            ms = [int(v) for v in p[:4]]
            K, N, al, be = int(p[4]), int(p[5]), p[6], p[7]
            A, B, C, ref = z[pre + "A"], z[pre + "B"], z[pre + "C"], z[pre + "out"]
            a_list, b_list, c_list, s = [], [], [], 0
            for g, mg in enumerate(ms):
                a_list.append(A[s:s + mg])
                bg = B[g * K:(g + 1) * K]
                b_list.append(np.ascontiguousarray(bg.T) if nk else bg)
                c_list.append(C[s:s + mg])
                s += mg
            # The golden vectors come from Triton's CPU interpreter, which evaluates
            # input_precision="tf32" dots in plain fp32: they pin layout, alpha/beta and the
            # epilogue of group_tf32gemm, not the TF32 rounding of the inputs.
            outs = go.group_gemm(kind, a_list, b_list, c_list, al, be, b_stored_nk=nk, tf32_mode="none")
            got = np.concatenate(outs, 0)
            assert not np.isnan(ref).any()
            tol = dict(rtol=1e-3, atol=1e-3) if kind == "fp16" else dict(rtol=2e-5, atol=2e-5)
            np.testing.assert_allclose(got, ref, err_msg=pre, **tol)
    C = go.group_mm("fp16", z["mm_A"], z["mm_B"], z["mm_offs"])
    np.testing.assert_allclose(C[:108], z["mm_C"][:108], rtol=1e-3, atol=1e-3)


def test_rounding_helpers():
    import torch

    x = torch.randn(20000) * 50
    assert np.array_equal(go.round_bf16(x.numpy()), x.bfloat16().float().numpy())
    assert np.array_equal(go.round_fp16(x.numpy()), x.half().float().numpy())
    t = go.trunc_tf32(x.numpy())
    r = go.round_tf32(x.numpy())
    assert np.all(np.abs(t) <= np.abs(x.numpy()))
    assert np.all(np.abs(r - x.numpy()) <= np.abs(t - x.numpy()) + 1e-12)
    assert np.all((t.view(np.uint32) & 0x1FFF) == 0) and np.all((r.view(np.uint32) & 0x1FFF) == 0)
