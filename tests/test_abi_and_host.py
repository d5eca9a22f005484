"""CPU-only checks: the C-ABI library loads and exports what the header declares,
host-side argument validation, the Python wrappers' error behaviour, and the
multi-GPU planning logic.  No kernel is launched."""
import ctypes
import os
import re

import pytest
import torch

import flagblas_b200 as fb
from flagblas_b200 import _lib, dist
from flagblas_b200.ops import CUBLAS_OP_N, CUBLAS_OP_T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flagblas_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    declared = _declared_symbols()
    assert "fb_gemm" in declared and "fb_group_gemm" in declared and "fb_group_mm" in declared
    handle = ctypes.CDLL(os.path.join(ROOT, "flagblas_b200", "libflagblas_b200.so"))
    for name in declared:
        assert hasattr(handle, name), name
    assert sorted(_lib.EXPORTED_SYMBOLS) == [d for d in declared if d in _lib.EXPORTED_SYMBOLS]
    missing_binding = [d for d in declared if d not in _lib.EXPORTED_SYMBOLS]
    assert missing_binding == [] or all(m.startswith("fb_") for m in missing_binding)


def test_status_strings():
    s = _lib.lib.fb_status_string
    assert s(0) == b"ok"
    assert b"invalid" in s(-1)
    assert b"workspace" in s(-2)
    assert b"timed out" in s(102)
    assert b"unknown" in s(12345)


def test_argument_validation_without_gpu():
    L = _lib.lib
    # rejected before any CUDA call is made
    assert L.fb_gemm(99, 0, 0, 8, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 8, None, 0, None) == -1   # dtype
    assert L.fb_gemm(_lib.FB_F16, 2, 0, 8, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 8, None, 0, None) == -1  # OP_C
    assert L.fb_gemm(_lib.FB_F16, 0, 0, -1, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 8, None, 0, None) == -1
    assert L.fb_gemm(_lib.FB_F16, 0, 0, 1 << 31, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 8, None, 0, None) == -4
    assert L.fb_gemm(_lib.FB_F16, 0, 0, 0, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 8, None, 0, None) == 0   # m == 0
    assert L.fb_gemm(_lib.FB_F16, 0, 0, 8, 8, 8, 1.0, None, 8, None, 8, 0.0, None, 4, None, 0, None) == -1  # ldc < n
    assert L.fb_group_gemm(_lib.FB_F32, 0, *([None] * 10), 4, 0, 0, 0, 1.0, 0.0, None, 0, None) == -1
    assert L.fb_group_gemm(_lib.FB_BF16, 0, *([None] * 10), 0, 0, 0, 0, 1.0, 0.0, None, 0, None) == 0
    assert L.fb_group_gemm(_lib.FB_BF16, 0, *([None] * 10), 4, 0, 0, 0, 1.0, 0.0, None, 0, None) == -1  # NULL arrays
    assert L.fb_selftest_bounded_wait(0, None) == -1
    # workspace sizing is pure host arithmetic
    assert L.fb_gemm_workspace_bytes(_lib.FB_F32, 0, 0, 100, 100, 100, 4, 101, 4, 101) == 0
    assert L.fb_gemm_workspace_bytes(_lib.FB_BF16, 0, 0, 128, 128, 128, 256, 128, 512, 128) == 0
    need = L.fb_gemm_workspace_bytes(_lib.FB_BF16, 0, 0, 100, 60, 50, 256, 51, 512, 64)  # lda*2 % 16 != 0
    assert need == ((100 * 56 * 2 + 255) // 256) * 256
    need = L.fb_gemm_workspace_bytes(_lib.FB_BF16, 0, 0, 100, 60, 50, 258, 56, 512, 64)  # A base misaligned
    assert need == ((100 * 56 * 2 + 255) // 256) * 256
    assert L.fb_group_workspace_bytes(0) == 0
    assert L.fb_group_workspace_bytes(64) >= 64 * 2 * 128 + 64 * 48


def test_wrappers_assert_like_the_reference():
    a = torch.zeros(8, 8)
    nc = torch.zeros(8, 16)[:, ::2]
    with pytest.raises(AssertionError):
        fb.sgemm(CUBLAS_OP_N, CUBLAS_OP_N, 8, 8, 8, 1.0, nc, 8, a, 8, 0.0, a.clone(), 8)   # non-contiguous
    with pytest.raises(AssertionError):
        fb.sgemm(CUBLAS_OP_N, CUBLAS_OP_N, 8, 8, 8, 1.0, a.half(), 8, a, 8, 0.0, a.clone(), 8)  # dtype
    with pytest.raises(AssertionError):
        fb.sgemm(2, CUBLAS_OP_N, 8, 8, 8, 1.0, a, 8, a, 8, 0.0, a.clone(), 8)  # CUBLAS_OP_C
    with pytest.raises(AssertionError):
        fb.hgemm(CUBLAS_OP_N, CUBLAS_OP_N, 8, 8, 8, 1.0, a, 8, a, 8, 0.0, a.clone(), 8)  # fp32 into hgemm
    # there is no CPU path: valid CPU tensors are refused loudly, not computed
    with pytest.raises(RuntimeError, match="no CPU path"):
        fb.sgemm(CUBLAS_OP_N, CUBLAS_OP_T, 8, 8, 8, 1.0, a, 8, a, 8, 0.0, a.clone(), 8)
    with pytest.raises(AssertionError):
        fb.group_mm(torch.zeros(4, 4, 4).half(), torch.zeros(2, 4, 4).half(), torch.zeros(2, dtype=torch.int32))


def test_api_surface():
    import flag_blas

    for name in ("sgemm", "hgemm", "bfgemm", "tf32gemm", "group_bfgemm", "group_hgemm", "group_tf32gemm",
                 "group_mm", "group_gemm"):
        assert callable(getattr(flag_blas, name)) and getattr(flag_blas, name) is getattr(fb, name)
    from flag_blas.ops import CUBLAS_OP_N as n_, CUBLAS_OP_T as t_  # noqa: F401
    assert (n_, t_, flag_blas.ops.CUBLAS_OP_C) == (0, 1, 2)
    assert flag_blas.device == "cuda" and flag_blas.vendor_name == "nvidia"
    assert flag_blas.runtime.device.support_bf16 and flag_blas.runtime.device.support_fp64
    assert flag_blas.testing.RESOLUTION[torch.bfloat16] == 0.016
    # the compiled module the reference reserves a hook for: a pybind11 binding of the same C ABI
    assert flag_blas.c_operators.__name__.endswith("c_operators") and callable(flag_blas.c_operators.gemm)
    assert flag_blas.c_operators.gemm(99, 0, 0, 8, 8, 8, 1.0, 0, 8, 0, 8, 0.0, 0, 8, 0, 0, 0) == -1
    assert flag_blas.c_operators.status_string(-6).startswith("request exceeds")
    import yaml
    ops = yaml.safe_load(open(os.path.join(ROOT, "conf", "operators.yaml")))
    ids = {o["id"] for o in ops["ops"]}
    assert {"sgemm", "hgemm", "bfgemm", "group_bfgemm", "group_hgemm", "group_tf32gemm", "group_mm"} <= ids


def test_column_ranges():
    assert dist.column_ranges(8192, 8) == [(i * 1024, (i + 1) * 1024) for i in range(8)]
    r = dist.column_ranges(14336, 4)
    assert r[0][0] == 0 and r[-1][1] == 14336 and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    assert all(s % 256 == 0 for s, _ in r)
    assert max(e - s for s, e in r) - min(e - s for s, e in r) <= 256
    r = dist.column_ranges(300, 4)
    assert r == [(0, 256), (256, 300), (300, 300), (300, 300)]
    assert dist.column_ranges(0, 2) == [(0, 0), (0, 0)]


def test_group_plan_balances_zipf():
    g = torch.Generator().manual_seed(3)
    w = torch.arange(1, 65, dtype=torch.float64) ** -1.2
    ms = torch.multinomial(w / w.sum(), 32768, replacement=True, generator=g).bincount(minlength=64).tolist()
    assert sum(ms) == 32768
    n, k = [1536] * 64, [4096] * 64
    for world in (1, 2, 4, 8):
        plan = dist.plan_group_shards(ms, n, k, world)
        # every row of every group is covered exactly once
        seen = {}
        for p in plan:
            for grp, s, rows in p:
                seen.setdefault(grp, []).append((s, rows))
        for grp, m in enumerate(ms):
            segs = sorted(seen.get(grp, []))
            pos = 0
            for s, rows in segs:
                assert s == pos
                pos += rows
            assert pos == m
        assert dist.plan_imbalance(plan, ms, n, k) < 1.03
    assert dist.plan_group_shards([0, 0], [8, 8], [8, 8], 2) == [[], []]


def test_shard_group_arrays_addresses():
    ms, n, k = [300, 0, 700], [64, 64, 64], [128, 128, 128]
    plan = dist.plan_group_shards(ms, n, k, 2, row_align=256)
    a = [1000, 2000, 3000]
    b = [10, 20, 30]
    o = [5000, 6000, 7000]
    rows_seen = {0: 0, 2: 0}
    for pieces in plan:
        (ap, bp, cp, op, m_, n_, k_, la, lb, lc), cnt = dist.shard_group_arrays(
            pieces, a, b, o, o, ms, n, k, k, n, n, 2, "cpu")
        assert cnt == len(pieces) and ap.dtype == torch.int64 and m_.dtype == torch.int32
        for i, (g, start, rows) in enumerate(pieces):
            assert int(ap[i]) == a[g] + start * k[g] * 2          # A advances by whole rows of lda elements
            assert int(bp[i]) == b[g]                              # B is shared by the slices of a group
            assert int(op[i]) == o[g] + start * n[g] * 2 and int(cp[i]) == int(op[i])
            assert int(m_[i]) == rows and int(n_[i]) == 64 and int(k_[i]) == 128
            rows_seen[g] += rows
    assert rows_seen == {0: 300, 2: 700}


def test_bench_reference_arm_prints_one_json_line():
    """`bench.py --impl reference` (the CPU arm) needs no GPU: stdout must be exactly one JSON line with the
    keys the harness reads."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--workload", "sgemm_512_nn"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-500:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "config",
                "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["value"] > 0 and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["config"]["workload"] == "sgemm_512_nn"
