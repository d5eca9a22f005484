"""Generate ``gpu_reference.npz``: outputs of the REFERENCE's own Triton kernels run natively on a GPU.

Complements ``make_golden.py`` (CPU interpreter: fp32 / fp16 only): on a GPU the reference's generic
level-3 kernels also run in bf16 and with real TF32 dots, which pins the two things the CPU vectors
cannot -- bfloat16 results and the TF32 rounding the reference's lowering applies.

Needs an installed copy of the reference (it is not shipped with this repo), e.g.

    python -m pip install --no-deps --no-build-isolation --target baseline/_ref /path/to/FlagBLAS
    FLAGBLAS_REFERENCE_SITE=baseline/_ref python tests/golden/make_golden_gpu.py          # gpu_reference.npz
    FLAGBLAS_REFERENCE_SITE=baseline/_ref python tests/golden/make_golden_gpu.py gemv     # gpu_reference_gemv.npz
    FLAGBLAS_REFERENCE_SITE=baseline/_ref python tests/golden/make_golden_gpu.py xgemm    # gpu_reference_xgemm.npz
    FLAGBLAS_REFERENCE_SITE=baseline/_ref python tests/golden/make_golden_gpu.py full_size  # gpu_reference_full_size.npz

and a CUDA device.  The same import shims as ``make_golden.py`` apply (stub ``sqlalchemy``,
``BLAS_VENDOR`` / ``ARCH`` / ``FLAGGEMS_DB_URL``, pass-through ``libentry`` that launches every kernel
with the first configuration of its tuning list); only the *generic* kernels of
``flag_blas.ops.level3`` and the kernels of ``flag_blas.ops.level2.gemv`` are called (plain pointer
kernels, one CTA per tile, no clusters).
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SITE = os.path.abspath(os.environ.get("FLAGBLAS_REFERENCE_SITE", os.path.join(ROOT, "baseline", "_ref")))


def _import_reference():
    os.environ.pop("TRITON_INTERPRET", None)
    os.environ["BLAS_VENDOR"] = "nvidia"
    os.environ["ARCH"] = "sm_90"
    os.environ["FLAGGEMS_DB_URL"] = "sqlite:////tmp/flagblas_golden_gpu.db"
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]  # the repo's own flag_blas alias must not win
    sys.path.insert(0, SITE)

    class _Any:
        def __init__(self, *a, **k):
            pass

        def __getattr__(self, n):
            return _Any()

        def __call__(self, *a, **k):
            return _Any()

        def __class_getitem__(cls, i):
            return cls

    sa = types.ModuleType("sqlalchemy")
    for sub in ("ext", "ext.automap", "orm", "exc", "engine", "schema"):
        sys.modules["sqlalchemy." + sub] = types.ModuleType("sqlalchemy." + sub)
    sys.modules["sqlalchemy"] = sa
    sa.ext = sys.modules["sqlalchemy.ext"]
    sa.ext.automap = sys.modules["sqlalchemy.ext.automap"]
    sa.orm, sa.exc = sys.modules["sqlalchemy.orm"], sys.modules["sqlalchemy.exc"]
    sa.engine, sa.schema = sys.modules["sqlalchemy.engine"], sys.modules["sqlalchemy.schema"]

    class DeclarativeBase:
        pass

    class Session:
        def __init__(self, *a, **k):
            pass

    sa.orm.DeclarativeBase, sa.orm.Session = DeclarativeBase, Session
    sa.orm.Mapped = sa.orm.MappedColumn = _Any
    sa.orm.mapped_column = lambda **k: None
    sa.exc.IntegrityError = Exception
    sa.engine.Engine = _Any
    sa.create_engine = lambda url: _Any()
    sa.ext.automap.AutomapBase = _Any

    class _AB:
        classes = {}

        def prepare(self, e):
            pass

    sa.ext.automap.automap_base = lambda: _AB()
    sa.inspect = lambda o: _Any()

    shim = types.ModuleType("flag_blas.utils.libentry")

    class _Tuned:
        def __init__(self, fn, configs):
            self.fn, self.configs = fn, configs

        def __getitem__(self, grid):
            cfg = self.configs[0]
            extra = dict(cfg.kwargs)
            extra.update(num_warps=cfg.num_warps, num_stages=cfg.num_stages)
            return lambda *a, **k: self.fn[grid](*a, **k, **extra)

    class _LC:
        model = None

    shim.libentry = lambda: (lambda fn: fn)
    shim.libtuner = lambda configs, key, **kw: (lambda fn: _Tuned(fn, configs))
    shim.libcache = _LC()
    sys.modules["flag_blas.utils.libentry"] = shim

    import torch
    import flag_blas  # noqa: F401  (the reference)

    assert os.path.abspath(flag_blas.__file__).startswith(SITE), flag_blas.__file__
    mods = {}
    for name in ("sgemm", "hgemm", "bfgemm"):
        mods[name] = getattr(sys.modules["flag_blas.ops.level3." + name], name)
    gg = sys.modules["flag_blas.ops.level3.group_gemm"]
    for name in ("group_bfgemm", "group_hgemm", "group_tf32gemm", "group_mm"):
        mods[name] = getattr(gg, name)
    gv = sys.modules["flag_blas.ops.level2.gemv"]
    for name in ("sgemv", "hgemv", "bfgemv", "fp8_gemv"):
        mods[name] = getattr(gv, name)
    for name in ("dgemm", "cgemm", "zgemm"):
        mods[name] = getattr(sys.modules["flag_blas.ops.level3." + name], name)
    for name in ("strmm", "dtrmm", "ctrmm", "ztrmm"):
        mods[name] = getattr(sys.modules["flag_blas.ops.level3.trmm"], name)
    return torch, mods


def main_xgemm():
    """``gpu_reference_xgemm.npz``: the reference's dgemm / cgemm / zgemm and strmm / dtrmm / ctrmm / ztrmm on the
    seeded cases."""
    torch, ref = _import_reference()
    sys.path.insert(0, HERE)
    import gpu_cases as gc

    dev = "cuda"
    out = {"device": np.array(torch.cuda.get_device_name(0)), "triton": np.array(__import__("triton").__version__)}
    for name in ("dgemm", "cgemm", "zgemm"):
        for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.xgemm_cases(name):
            Cd = C.to(dev)
            ref[name](ta, tb, m, n, k, alpha, A.to(dev), lda, B.to(dev), ldb, beta, Cd, ldc)
            torch.cuda.synchronize()
            out[key + "_C"] = Cd.cpu().numpy()
            out[key + "_probe"] = np.concatenate([A.numpy().ravel()[:4], B.numpy().ravel()[:4]])
        print(name, "done", flush=True)
    for name in ("strmm", "dtrmm", "ctrmm", "ztrmm"):
        for key, (side, uplo, trans, diag, m, n, lda, ldb, ldc, alpha), A, B, C in gc.trmm_cases(name):
            Cd = C.to(dev)
            ref[name](side, uplo, trans, diag, m, n, alpha, A.to(dev), lda, B.to(dev), ldb, Cd, ldc)
            torch.cuda.synchronize()
            out[key + "_C"] = Cd.cpu().numpy()
            out[key + "_probe"] = np.concatenate([A.numpy().ravel()[:4], B.numpy().ravel()[:4]])
        print(name, "done", flush=True)
    path = os.path.join(HERE, "gpu_reference_xgemm.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_gemv():
    """``gpu_reference_gemv.npz``: the reference's sgemv / hgemv / bfgemv on the seeded cases of gpu_cases."""
    torch, ref = _import_reference()
    sys.path.insert(0, HERE)
    import gpu_cases as gc

    dev = "cuda"
    out = {"device": np.array(torch.cuda.get_device_name(0)), "triton": np.array(__import__("triton").__version__)}
    for name in ("sgemv", "hgemv", "bfgemv"):
        for key, (trans, m, n, lda, incx, incy, alpha, beta), A, x, y in gc.gemv_cases(name):
            yd = y.to(dev)
            ref[name](trans, m, n, alpha, A.to(dev), lda, x.to(dev), incx, beta, yd, incy)
            torch.cuda.synchronize()
            out[key + "_y"] = gc.pack(yd.cpu())
            out[key + "_probe"] = np.concatenate([A.float().numpy().ravel()[:8], x.float().numpy().ravel()[:1]])
        print("gemv", name, "done", flush=True)
    for key, (m, n, lda, incx, incy, ky, alpha, beta), A, x, y in gc.fp8_gemv_cases():
        yd = y.to(dev)
        # the reference asserts lda == A.stride(0): hand it the padded matrix as a column slice
        ref["fp8_gemv"](1, m, n, alpha, A.to(dev)[:, :n], lda, x.to(dev), incx, beta, yd, incy)
        torch.cuda.synchronize()
        out[key + "_y"] = gc.pack(yd.cpu())
        out[key + "_probe"] = np.concatenate([A.float().numpy().ravel()[:8], x.float().numpy().ravel()[:1]])
    print("fp8_gemv done", flush=True)
    path = os.path.join(HERE, "gpu_reference_gemv.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def main():
    torch, ref = _import_reference()
    sys.path.insert(0, HERE)
    import gpu_cases as gc

    dev = "cuda"
    out = {"device": np.array(torch.cuda.get_device_name(0)), "triton": np.array(__import__("triton").__version__)}
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731

    # ---------------------------------------------------------------- dense bf16 / fp16 / fp32
    for kind, fn in (("bf16", ref["bfgemm"]), ("fp16", ref["hgemm"]), ("fp32", ref["sgemm"])):
        for key, (ta, tb, m, n, k, lda, ldb, ldc, alpha, beta), A, B, C in gc.dense_cases(kind):
            Cd = C.to(dev)
            fn(ta, tb, m, n, k, alpha, A.to(dev), lda, B.to(dev), ldb, beta, Cd, ldc)
            torch.cuda.synchronize()
            out[key + "_C"] = gc.pack(Cd.cpu())
            out[key + "_probe"] = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
        print("dense", kind, "done", flush=True)

    # ---------------------------------------------------------------- grouped bf16 / fp16 / tf32
    for kind, fn, transB in (("bf16", ref["group_bfgemm"], False), ("fp16", ref["group_hgemm"], False),
                             ("tf32", ref["group_tf32gemm"], True)):
        for tag in ("ab", "b0"):
            ms, K, N, al, be, A, B, C = gc.group_case(kind, tag)
            E = len(ms)
            Ad, Cd = A.to(dev), C.to(dev)
            o = torch.full_like(Cd, float("nan")) if be == 0.0 else torch.zeros_like(Cd)
            Bs = (torch.cat([B[g * K:(g + 1) * K].t().contiguous() for g in range(E)], 0) if transB else B).to(dev)
            es = A.element_size()
            ap, bp, cp, op, s = [], [], [], [], 0
            for g, mg in enumerate(ms):
                ap.append(Ad.data_ptr() + s * K * es); cp.append(Cd.data_ptr() + s * N * es)
                op.append(o.data_ptr() + s * N * es); bp.append(Bs.data_ptr() + g * K * N * es)
                s += mg
            fn(o, i64(ap), i64(bp), i64(cp), i64(op), i32(ms), i32([N] * E), i32([K] * E), i32([K] * E),
               i32([K if transB else N] * E), i32([N] * E), E, sum(ms), N, K, alpha=al, beta=be)
            torch.cuda.synchronize()
            out["group_%s_%s_out" % (kind, tag)] = gc.pack(o.cpu())
            out["group_%s_%s_probe" % (kind, tag)] = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
        print("grouped", kind, "done", flush=True)

    # TF32 rounding probe through the reference's group_tf32gemm (one group)
    m, n, k, A, Bt = gc.tf32_probe()
    Ad, Bd = A.to(dev), Bt.to(dev)
    o = torch.zeros(m, n, device=dev)
    ref["group_tf32gemm"](o, i64([Ad.data_ptr()]), i64([Bd.data_ptr()]), i64([o.data_ptr()]), i64([o.data_ptr()]), i32([m]), i32([n]),
                          i32([k]), i32([k]), i32([k]), i32([n]), 1, m, n, k, alpha=1.0, beta=0.0)
    torch.cuda.synchronize()
    out["tf32probe_out"] = o.cpu().numpy()

    A, B, offs = gc.group_mm_case()
    Cm = ref["group_mm"](A.to(dev), B.to(dev), offs.to(dev))
    torch.cuda.synchronize()
    out["mm_C"] = gc.pack(Cm.cpu())

    path = os.path.join(HERE, "gpu_reference.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_full_size():
    """``gpu_reference_full_size.npz``: samples (whole rows and whole columns) of what the reference's generic
    kernels give on the benchmark workloads at full size: fp16 8192^3, the bf16 MLP shape with beta = 1, the 64-expert
    MoE, and the two TF32 contractions (the reference has TF32 only in grouped form, so those run as a single group
    of ``group_tf32gemm`` on operands laid out the way it wants them: A as [m, k], B as [n, k])."""
    torch, ref = _import_reference()
    sys.path.insert(0, HERE)
    import gpu_cases as gc

    dev = "cuda"
    out = {"device": np.array(torch.cuda.get_device_name(0)), "triton": np.array(__import__("triton").__version__)}
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    for name in gc.FULL_SIZE:
        kind, ta, tb, m, n, k, alpha, beta, A, B, C = gc.full_size_dense(name)
        rows, cols = gc.sample_rows_cols(m, n)
        Ad, Bd, Cd = A.to(dev), B.to(dev), C.to(dev)
        if kind == "tf32":
            Am = Ad.t().contiguous() if ta else Ad           # [m, k]
            Bn = Bd if tb else Bd.t().contiguous()           # [n, k]
            o = torch.empty_like(Cd)
            ref["group_tf32gemm"](o, i64([Am.data_ptr()]), i64([Bn.data_ptr()]), i64([Cd.data_ptr()]), i64([o.data_ptr()]),
                                  i32([m]), i32([n]), i32([k]), i32([k]), i32([k]), i32([n]), 1, m, n, k, alpha=alpha, beta=beta)
            res = o
        else:
            if beta == 0.0:
                Cd.fill_(float("nan"))
            fn = ref["hgemm"] if kind == "fp16" else ref["bfgemm"]
            fn(ta, tb, m, n, k, alpha, Ad, A.shape[1], Bd, B.shape[1], beta, Cd, n)
            res = Cd
        torch.cuda.synchronize()
        out[name + "_rows"] = np.array(rows)
        out[name + "_cols"] = np.array(cols)
        out[name + "_row_vals"] = gc.pack(res[rows].cpu())
        out[name + "_col_vals"] = gc.pack(res[:, cols].cpu())
        out[name + "_probe"] = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
        print("full size", name, "done", flush=True)
        del Ad, Bd, Cd, res

    ms, K, N, A, B = gc.moe_case()
    E = len(ms)
    Ad, Bd = A.to(dev), B.to(dev)
    o = torch.full((sum(ms), N), float("nan"), dtype=torch.bfloat16, device=dev)
    ap, bp, op, s = [], [], [], 0
    for g, mg in enumerate(ms):
        ap.append(Ad.data_ptr() + s * K * 2); op.append(o.data_ptr() + s * N * 2); bp.append(Bd.data_ptr() + g * K * N * 2)
        s += mg
    ref["group_bfgemm"](o, i64(ap), i64(bp), i64(op), i64(op), i32(ms), i32([N] * E), i32([K] * E), i32([K] * E),
                        i32([N] * E), i32([N] * E), E, sum(ms), N, K, alpha=1.0, beta=0.0)
    torch.cuda.synchronize()
    rows, s = [], 0
    for mg in ms:            # first and last token of every expert
        if mg:
            rows += sorted({s, s + mg - 1})
        s += mg
    out["moe_ms"] = np.array(ms)
    out["moe_rows"] = np.array(rows)
    out["moe_row_vals"] = gc.pack(o[rows].cpu())
    out["moe_col_vals"] = gc.pack(o[:, gc.MOE_COLS].cpu())
    out["moe_probe"] = np.concatenate([A.float().numpy().ravel()[:8], B.float().numpy().ravel()[:8]])
    print("full size moe done", flush=True)
    path = os.path.join(HERE, "gpu_reference_full_size.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if sys.argv[1:] == ["full_size"]:
        main_full_size()
    elif sys.argv[1:] == ["gemv"]:
        main_gemv()
    elif sys.argv[1:] == ["xgemm"]:
        main_xgemm()
    else:
        main()
