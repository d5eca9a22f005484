"""The dense kernel's alternative configurations (single-CTA tiles, 2-D copies, one k-slab per stage,
narrow tiles) must compute the same results as the default plan."""
import pytest
import torch

import flagblas_b200 as fb
from tests.helpers import KINDS, assert_parity, make_dense, oracle_dense, result_scale

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("env", [{"FLAGBLAS_B200_PAIR": "0"}, {"FLAGBLAS_B200_TMA3D": "0"}, {"FLAGBLAS_B200_KS": "1"},
                                 {"FLAGBLAS_B200_BLOCK_N": "128"}, {"FLAGBLAS_B200_PAIR": "0", "FLAGBLAS_B200_BLOCK_N": "64"},
                                 {"FLAGBLAS_B200_STAGES": "2"}, {"FLAGBLAS_B200_GROUP_M": "3"}])
@pytest.mark.parametrize("kind", ["bf16", "tf32"])
def test_dense_plan_variants(env, kind, monkeypatch):
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
        m, n, k = 640, 896, 448
        A, lda, B, ldb, C, ldc = make_dense(kind, ta, tb, m, n, k, seed=21)
        ref = oracle_dense(kind, ta, tb, m, n, k, 1.5, A, lda, B, ldb, 0.5, C, ldc)
        Cd = C.to(DEV)
        getattr(fb, KINDS[kind][1])(ta, tb, m, n, k, 1.5, A.to(DEV), lda, B.to(DEV), ldb, 0.5, Cd, ldc)
        torch.cuda.synchronize()
        assert fb.device_status() == 0
        assert_parity(Cd.float().cpu(), ref, KINDS[kind][2], result_scale(k, A, B, 1.5) + 0.5, "%s %s ta=%d tb=%d" % (kind, env, ta, tb))
