"""``flag_blas.use_blas()``: aten::mm / addmm / bmm / mv / addmv served by this library (reference
scaffolding: src/flag_blas/__init__.py:49-189).  CPU part: table and stride logic.  GPU part: results
inside the context against torch's own kernels outside it, and proof that the override really ran."""
import pytest
import torch

import flagblas_b200 as fb
from flagblas_b200 import aten


def test_table_and_registrar_selection():
    assert [item[0] for item in aten._FULL_CONFIG] == ["mm", "addmm", "bmm", "mv", "addmv", "_grouped_mm"]

    class FakeLib:
        def __init__(self):
            self.calls = []

        def impl(self, key, fn, dispatch_key):
            self.calls.append((key, fn.__name__, dispatch_key))

    lib = FakeLib()
    r = aten.Register(aten._FULL_CONFIG, user_exclude_ops=["bmm", "addmv"], lib=lib)
    assert r.get_all_keys() == ["mm", "addmm", "mv", "_grouped_mm"] and all(c[2] == "CUDA" for c in lib.calls)
    lib = FakeLib()
    r = aten.Register(aten._FULL_CONFIG, user_include_ops=["mv"], lib=lib)
    assert r.get_all_ops() == ["mv"]
    with pytest.raises(ValueError):
        aten.Register(aten._FULL_CONFIG, lib=None)


def test_as_operand_strides():
    a = torch.zeros(6, 8)
    t, trans, ld = aten.as_operand(a)
    assert (trans, ld) == (0, 8) and t.data_ptr() == a.data_ptr()
    t, trans, ld = aten.as_operand(a.t())                 # stored [6, 8], seen as [8, 6]
    assert (trans, ld) == (1, 8) and t.data_ptr() == a.data_ptr()
    t, trans, ld = aten.as_operand(a[:, :5])              # row-major with pitch 8
    assert (trans, ld) == (0, 8)
    t, trans, ld = aten.as_operand(a[::2, ::2])           # neither: copied
    assert (trans, ld) == (0, 4) and t.is_contiguous()
    t, trans, ld = aten.as_operand(torch.zeros(1, 8).expand(4, 8))
    assert (trans, ld) == (0, 8) and t.is_contiguous()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_use_blas_serves_torch_matmul(dtype, monkeypatch):
    dev = "cuda"
    g = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randn(300, 200, generator=g).to(dtype).to(dev)
    b = torch.randn(200, 136, generator=g).to(dtype).to(dev)
    bt = torch.randn(136, 200, generator=g).to(dtype).to(dev)
    bias = torch.randn(136, generator=g).to(dtype).to(dev)
    x = torch.randn(200, generator=g).to(dtype).to(dev)
    ba = torch.randn(3, 64, 200, generator=g).to(dtype).to(dev)
    bb = torch.randn(3, 200, 72, generator=g).to(dtype).to(dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    want = [torch.mm(a, b), a @ bt.t(), torch.addmm(bias, a, b, beta=0.5, alpha=2.0), torch.bmm(ba, bb),
            torch.mv(a, x), torch.mv(a.t(), torch.mv(a, x)), torch.addmv(torch.mv(a, x), a, x, beta=0.5, alpha=-1.0),
            torch.nn.functional.linear(a, bt, bias)]
    calls = {"gemm": 0, "gemv": 0}
    real_gemm, real_gemv = aten._gemm._launch, aten._gemv._call
    monkeypatch.setattr(aten._gemm, "_launch", lambda *p: (calls.__setitem__("gemm", calls["gemm"] + 1), real_gemm(*p))[1])
    monkeypatch.setattr(aten._gemv, "_call", lambda *p: (calls.__setitem__("gemv", calls["gemv"] + 1), real_gemv(*p))[1])
    with fb.use_blas():
        assert fb.all_registered_keys() == ["mm", "addmm", "bmm", "mv", "addmv", "_grouped_mm"]
        got = [torch.mm(a, b), a @ bt.t(), torch.addmm(bias, a, b, beta=0.5, alpha=2.0), torch.bmm(ba, bb),
               torch.mv(a, x), torch.mv(a.t(), torch.mv(a, x)), torch.addmv(torch.mv(a, x), a, x, beta=0.5, alpha=-1.0),
               torch.nn.functional.linear(a, bt, bias)]
        torch.cuda.synchronize()
        inside = dict(calls)
    assert inside["gemm"] >= 3 and inside["gemv"] >= 5
    assert fb.all_registered_keys() == []
    torch.mm(a, b)                                       # the library is gone: torch's own kernel again
    assert calls == inside
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for w, gv in zip(want, got):
        assert w.shape == gv.shape and w.dtype == gv.dtype
        scale = float(w.float().abs().max())
        assert float((w.float() - gv.float()).abs().max()) <= tol * scale * (4 if len(w.shape) == 1 else 1)
    assert fb.device_status() == 0


@pytest.mark.gpu
def test_use_blas_autograd_and_include():
    dev = "cuda"
    a = torch.randn(64, 96, device=dev, requires_grad=True)
    b = torch.randn(96, 32, device=dev, requires_grad=True)
    (a @ b).sum().backward()
    ga, gb = a.grad.clone(), b.grad.clone()
    a.grad = b.grad = None
    with fb.use_blas(include=["mm"]):
        assert fb.all_registered_ops() == ["mm"]
        (a @ b).sum().backward()
    torch.testing.assert_close(a.grad, ga, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(b.grad, gb, rtol=1e-5, atol=1e-4)


@pytest.mark.gpu
def test_use_blas_double_and_complex():
    """After enable() / inside use_blas() every CUDA mm is overridden, so float64 and complex matrices must keep
    working: they run on the library's dgemm / cgemm / zgemm kernels."""
    dev = "cuda"
    g = torch.Generator(device="cpu").manual_seed(5)
    for dt, tol in ((torch.float64, 1e-12), (torch.complex64, 1e-5), (torch.complex128, 1e-12)):
        a = torch.randn(70, 96, generator=g, dtype=dt).to(dev)
        b = torch.randn(96, 40, generator=g, dtype=dt).to(dev)
        c = torch.randn(70, 40, generator=g, dtype=dt).to(dev)
        v = torch.randn(96, generator=g, dtype=dt).to(dev)
        bt = torch.randn(40, 96, generator=g, dtype=dt).to(dev)
        want = [a @ b, torch.addmm(c, a, b, beta=0.5, alpha=2.0), a @ bt.t(), torch.mv(a, v),
                torch.bmm(torch.stack([a, a]), torch.stack([b, b]))]
        if dt.is_complex:
            want.append(a @ bt.mH)
        with fb.use_blas():
            got = [a @ b, torch.addmm(c, a, b, beta=0.5, alpha=2.0), a @ bt.t(), torch.mv(a, v),
                   torch.bmm(torch.stack([a, a]), torch.stack([b, b]))]
            if dt.is_complex:
                got.append(a @ bt.mH)
            torch.cuda.synchronize()
        for w, gv in zip(want, got):
            assert w.shape == gv.shape and w.dtype == gv.dtype
            assert float((w - gv).abs().max()) <= tol * 96 ** 0.5 * 4, dt
    with fb.use_blas():
        with pytest.raises((NotImplementedError, RuntimeError)):
            torch.mm(torch.ones(4, 4, device=dev, dtype=torch.int32), torch.ones(4, 4, device=dev, dtype=torch.int32))
    assert fb.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_bmm_runs_as_one_grouped_launch(dtype, monkeypatch):
    """Aligned tensor-core batches go through group_mm (one launch for the whole batch); the fp32 IEEE case,
    unaligned rows and transposed batch entries fall back to, or are handled by, the per-entry path."""
    dev = "cuda"
    g = torch.Generator(device="cpu").manual_seed(2)
    a = torch.randn(12, 96, 64, generator=g).to(dtype).to(dev)
    b = torch.randn(12, 64, 136, generator=g).to(dtype).to(dev)
    bt = torch.randn(12, 136, 64, generator=g).to(dtype).to(dev)
    odd = torch.randn(12, 64, 33, generator=g).to(dtype).to(dev)
    torch.backends.cuda.matmul.allow_tf32 = dtype == torch.float32
    want = [torch.bmm(a, b), torch.bmm(a, bt.transpose(1, 2)), torch.bmm(a, odd)]
    import importlib
    gg = importlib.import_module("flagblas_b200.ops.level3.group_gemm")
    calls = {"n": 0}
    real = gg.group_mm
    monkeypatch.setattr(gg, "group_mm", lambda *p: (calls.__setitem__("n", calls["n"] + 1), real(*p))[1])
    with fb.use_blas(include=["bmm", "_grouped_mm"]):
        got = [torch.bmm(a, b), torch.bmm(a, bt.transpose(1, 2)), torch.bmm(a, odd)]
        offs = torch.tensor([96, 96, 500, 1152], dtype=torch.int32, device=dev)
        if dtype != torch.float32:
            gm = torch.ops.aten._grouped_mm(a.reshape(-1, 64), b[:4], offs)
            ref = torch.cat([a.reshape(-1, 64)[s:e].float() @ b[i].float() for i, (s, e) in
                             enumerate([(0, 96), (96, 96), (96, 500), (500, 1152)])])
            assert float((gm.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
        torch.cuda.synchronize()
    torch.backends.cuda.matmul.allow_tf32 = False
    assert calls["n"] >= 2
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    for w, gv in zip(want, got):
        assert w.shape == gv.shape
        assert float((w.float() - gv.float()).abs().max()) <= tol * float(w.float().abs().max())
    assert fb.device_status() == 0
