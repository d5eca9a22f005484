"""Generate the golden vectors in this directory by running the REFERENCE's own kernels.

Run where the reference checkout is available (it is not shipped with this repo):

    FLAGBLAS_REFERENCE=/path/to/FlagBLAS python tests/golden/make_golden.py

The reference is pure Python + Triton.  Without a GPU its generic level-3 kernels
run under Triton's CPU interpreter (``TRITON_INTERPRET=1``), which is how the
vectors below were made.  fp32 and fp16 work there; bf16 does not (the
interpreter has no bfloat16), so bf16 has no golden vector and is pinned through
the fp16 cases, whose code path differs from bf16 only in the final rounding.

The import needs four shims (none of them touches arithmetic):
  * a stub ``sqlalchemy`` (autotune persistence; absent here),
  * ``BLAS_VENDOR=nvidia``, ``ARCH=sm_90``, ``FLAGGEMS_DB_URL`` set,
  * ``flag_blas.utils.libentry`` replaced by a pass-through that launches each
    kernel with the first configuration of its tuning list,
  * the ``torch_device_fn`` device guard replaced by a null context.

Outputs: ``dense_fp32.npz``, ``dense_fp16.npz``, ``edge_fp32.npz``,
``config1_sgemm512.npz``, ``grouped.npz`` -- inputs, call parameters and the
reference's outputs, a few hundred KB in total.
"""
import contextlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("FLAGBLAS_REFERENCE")  # checkout of the reference project (its `src/` is put on sys.path)
if not REF:
    raise SystemExit("set FLAGBLAS_REFERENCE to a checkout of flagos-ai/FlagBLAS")


def _import_reference():
    os.environ["TRITON_INTERPRET"] = "1"
    os.environ["BLAS_VENDOR"] = "nvidia"
    os.environ["ARCH"] = "sm_90"
    os.environ["FLAGGEMS_DB_URL"] = "sqlite:////tmp/flagblas_golden.db"
    sys.path.insert(0, os.path.join(REF, "src"))

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
            return lambda *a, **k: self.fn[grid](*a, **k, **cfg.kwargs)

    class _LC:
        model = None

    shim.libentry = lambda: (lambda fn: fn)
    shim.libtuner = lambda configs, key, **kw: (lambda fn: _Tuned(fn, configs))
    shim.libcache = _LC()
    sys.modules["flag_blas.utils.libentry"] = shim

    import torch
    import flag_blas  # noqa: F401  (the reference)

    class _Dev:
        @staticmethod
        def device(d):
            return contextlib.nullcontext()

    mods = {}
    for name in ("sgemm", "hgemm", "bfgemm"):
        mod = sys.modules["flag_blas.ops.level3." + name]
        mod.torch_device_fn = _Dev
        mods[name] = getattr(mod, name)
    gg = sys.modules["flag_blas.ops.level3.group_gemm"]
    torch.cuda.get_device_properties = lambda *a, **k: types.SimpleNamespace(multi_processor_count=4)
    mods["group_hgemm"], mods["group_tf32gemm"], mods["group_mm"] = gg.group_hgemm, gg.group_tf32gemm, gg.group_mm
    return torch, mods


def main():
    torch, ref = _import_reference()
    gen = torch.Generator(device="cpu")

    # ---------------------------------------------------------------- dense
    for kind, fn, dt, ab in (("fp32", ref["sgemm"], torch.float32, (2.5, 0.5)),
                             ("fp16", ref["hgemm"], torch.float16, (1.5, 0.5))):
        out = {}
        gen.manual_seed(11)
        for ta in (0, 1):
            for tb in (0, 1):
                for ci, (m, n, k, pad) in enumerate(((96, 80, 72, 0), (70, 130, 45, 3))):
                    lda = (m if ta else k) + pad
                    ldb = (k if tb else n) + pad
                    ldc = n + pad
                    A = torch.randn((k if ta else m), lda, generator=gen).to(dt)
                    B = torch.randn((n if tb else k), ldb, generator=gen).to(dt)
                    C = torch.randn(m, ldc, generator=gen).to(dt)
                    C0 = C.clone()
                    fn(ta, tb, m, n, k, ab[0], A, lda, B, ldb, ab[1], C, ldc)
                    key = "t%d%d_c%d" % (ta, tb, ci)
                    out[key + "_A"], out[key + "_B"] = A.float().numpy(), B.float().numpy()
                    out[key + "_C0"], out[key + "_C"] = C0.float().numpy(), C.float().numpy()
                    out[key + "_p"] = np.array([ta, tb, m, n, k, lda, ldb, ldc, ab[0], ab[1]], dtype=np.float64)
        np.savez_compressed(os.path.join(HERE, "dense_%s.npz" % kind), **out)
        print("dense", kind, len(out) // 5, "cases")

    # ----------------------------------------------------------- edge cases
    out = {}
    gen.manual_seed(12)
    sg = ref["sgemm"]
    m = n = k = 64
    A = torch.randn(m, k, generator=gen)
    B = torch.randn(k, n, generator=gen)
    C = torch.randn(m, n, generator=gen)
    out["A"], out["B"], out["C0"] = A.numpy(), B.numpy(), C.numpy()
    c = C.clone(); sg(0, 0, m, n, k, 0.0, A, k, B, n, 0.5, c, n); out["alpha_zero"] = c.numpy()
    c = torch.full_like(C, float("nan")); sg(0, 0, m, n, k, 2.5, A, k, B, n, 0.0, c, n); out["beta_zero_nanC"] = c.numpy()
    c = C[:1].clone().contiguous(); sg(0, 0, 0, 64, 64, 2.5, A, 64, B, 64, 0.5, c, 64); out["empty_m0"] = c.numpy()
    c = C.clone(); sg(0, 0, 64, 64, 0, 2.5, A, 64, B, 64, 0.5, c, 64); out["empty_k0"] = c.numpy()
    c = C.clone(); sg(0, 0, 64, 0, 64, 2.5, A, 64, B, 64, 0.0, c, 64); out["empty_n0_beta0"] = c.numpy()
    for i, (al, be) in enumerate(((1.0, 0.0), (0.0, 1.0), (1.0, 1.0), (-1.0, 0.5), (2.5, -0.5))):
        c = C.clone(); sg(0, 0, m, n, k, al, A, k, B, n, be, c, n); out["ab%d" % i] = c.numpy()
        out["ab%d_p" % i] = np.array([al, be])
    np.savez_compressed(os.path.join(HERE, "edge_fp32.npz"), **out)
    print("edge done")

    # ------------------------------------------- the small fp32 benchmark workload: sgemm 512^3
    gen.manual_seed(0)
    m = n = k = 512
    A = torch.rand(m, k, generator=gen) * 2 - 1
    B = torch.rand(k, n, generator=gen) * 2 - 1
    C = torch.zeros(m, n)
    sg(0, 0, m, n, k, 1.0, A, k, B, n, 0.0, C, n)
    np.savez_compressed(os.path.join(HERE, "config1_sgemm512.npz"), A_probe=A[:4, :8].numpy(), B_probe=B[:4, :8].numpy(),
                        C_sub=C[::4, ::4].contiguous().numpy(), C_sum=np.array(C.double().sum().item()))
    print("config1 done")

    # -------------------------------------------------------------- grouped
    out = {}
    i32 = lambda l: torch.tensor(l, dtype=torch.int32)  # noqa: E731
    ms = [5, 0, 70, 33]
    K, N = 64, 48
    E = len(ms)
    for name, fn, dt, transB in (("h", ref["group_hgemm"], torch.float16, False),
                                 ("tf32", ref["group_tf32gemm"], torch.float32, True)):
        for tag, (al, be) in (("ab", (1.5, 0.5)), ("b0", (1.0, 0.0))):
            gen.manual_seed(13)
            A = torch.randn(sum(ms), K, generator=gen).to(dt)
            B = (torch.randn(E * K, N, generator=gen) * K ** -0.5).to(dt)
            C = torch.randn(sum(ms), N, generator=gen).to(dt)
            o = torch.full_like(C, float("nan")) if be == 0.0 else torch.zeros_like(C)
            Bs = torch.cat([B[g * K:(g + 1) * K].t().contiguous() for g in range(E)], 0) if transB else B
            ap, bp, cp, op, s = [], [], [], [], 0
            es = A.element_size()
            for g, mg in enumerate(ms):
                ap.append(A.data_ptr() + s * K * es)
                cp.append(C.data_ptr() + s * N * es)
                op.append(o.data_ptr() + s * N * es)
                bp.append(Bs.data_ptr() + g * K * N * es)
                s += mg
            fn(o, torch.tensor(ap), torch.tensor(bp), torch.tensor(cp), torch.tensor(op), i32(ms), i32([N] * E),
               i32([K] * E), i32([K] * E), i32([K if transB else N] * E), i32([N] * E), E, sum(ms), N, K,
               alpha=al, beta=be)
            pre = "g%s_%s_" % (name, tag)
            out[pre + "A"], out[pre + "B"], out[pre + "C"], out[pre + "out"] = (A.float().numpy(), B.float().numpy(),
                                                                                C.float().numpy(), o.float().numpy())
            out[pre + "p"] = np.array(ms + [K, N, al, be], dtype=np.float64)
    gen.manual_seed(14)
    A = torch.randn(108, 64, generator=gen).half()
    B = torch.randn(4, 64, 48, generator=gen).half()
    offs = torch.tensor([5, 5, 75, 108], dtype=torch.int32)
    Cm = ref["group_mm"](A, B, offs)
    out["mm_A"], out["mm_B"], out["mm_offs"], out["mm_C"] = A.float().numpy(), B.float().numpy(), offs.numpy(), Cm.float().numpy()
    np.savez_compressed(os.path.join(HERE, "grouped.npz"), **out)
    print("grouped done")


if __name__ == "__main__":
    main()
