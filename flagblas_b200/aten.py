"""``torch``-level entry: serve ``aten::mm / addmm / bmm / mv / addmv`` on CUDA tensors with this library.

Mirrors the registration scaffolding of the reference (``src/flag_blas/__init__.py:49-189``: ``enable``,
``only_enable``, ``use_blas``, ``all_registered_ops``, ``all_registered_keys``; ``runtime/register.py:21-145``:
the ``Register`` class walking a ``(aten key, function[, condition])`` table).  In the reference the table
(``_FULL_CONFIG``) is empty, so nothing is ever registered; here it lists the operators below.

The functions take whatever strides ``torch`` hands them: a matrix that is row-major, or the transpose
of a row-major matrix, is passed in place with ``trans = N / T`` and its pitch as the leading dimension;
anything else is made contiguous first.  fp16 and bf16 run on the tensor cores with fp32 accumulation;
fp32 runs the IEEE kernel unless ``torch.backends.cuda.matmul.allow_tf32`` is set, then the TF32 kernel.
float64, complex64 and complex128 go to the library's ``dgemm`` / ``cgemm`` / ``zgemm`` kernels (``fb_gemm_ex``).
Any other dtype raises ``NotImplementedError`` (torch's own CUDA ``mm`` has no integer or fp8 kernels either).
"""
import warnings

import torch

from . import _lib
from .ops._constants import CUBLAS_OP_N, CUBLAS_OP_T
from .ops.level2 import gemv as _gemv
from .ops.level3 import gemm as _gemm

_cop = _lib.cop


def _code(dtype):
    if dtype == torch.float16:
        return _lib.FB_F16
    if dtype == torch.bfloat16:
        return _lib.FB_BF16
    if dtype == torch.float32:
        return _lib.FB_TF32 if torch.backends.cuda.matmul.allow_tf32 else _lib.FB_F32
    raise NotImplementedError("flag_blas aten overrides cover float16, bfloat16, float32, float64, complex64 and "
                              "complex128, not %s" % dtype)


_EX_CODES = {torch.float64: _lib.FB_F64, torch.complex64: _lib.FB_C64, torch.complex128: _lib.FB_C128}


def _parts(v):
    v = complex(v.item() if isinstance(v, torch.Tensor) else v)
    return float(v.real), float(v.imag)


def _mm_into_ex(out, a, b, alpha, beta):
    """float64 / complex: out[m, n] (contiguous) <- alpha * a @ b + beta * out through ``fb_gemm_ex``."""
    m, k = a.shape
    n = b.shape[1]
    # a lazily conjugated view (x.mH, x.conj()) is materialised: the kernel sees plain memory
    a, ta, lda = as_operand(a.resolve_conj())
    b, tb, ldb = as_operand(b.resolve_conj())
    ar, ai = _parts(alpha)
    br, bi = _parts(beta)
    stream, prev = _lib.enter(out.device)
    try:
        status = _cop.gemm_ex(_EX_CODES[out.dtype], ta, tb, m, n, k, ar, ai, a.data_ptr(), lda, b.data_ptr(), ldb, br, bi,
                              out.data_ptr(), n, stream)
    finally:
        _lib.leave(prev)
    _lib.check(status, "aten::mm")
    return out


def as_operand(t):
    """``(tensor, trans, ld)`` with ``op(row-major [rows, ld] storage at tensor.data_ptr()) == t``."""
    r, c = t.shape
    if r > 1 and c > 1:
        if t.stride(1) == 1 and t.stride(0) >= c:
            return t, CUBLAS_OP_N, t.stride(0)
        if t.stride(0) == 1 and t.stride(1) >= r:
            return t, CUBLAS_OP_T, t.stride(1)
    t = t.contiguous()
    return t, CUBLAS_OP_N, max(c, 1)


def _mm_into(out, a, b, alpha, beta):
    """out[m, n] (contiguous) <- alpha * a @ b + beta * out."""
    m, k = a.shape
    n = b.shape[1]
    if m == 0 or n == 0:
        return out
    if k == 0:
        return out.zero_() if beta == 0 else out.mul_(beta)
    if out.dtype in _EX_CODES:
        return _mm_into_ex(out, a, b, alpha, beta)
    a, ta, lda = as_operand(a)
    b, tb, ldb = as_operand(b)
    _gemm._launch(_code(a.dtype), "aten::mm", ta, tb, m, n, k, float(alpha), a.data_ptr(), lda, b.data_ptr(), ldb,
                  float(beta), out.data_ptr(), n, a.device)
    return out


def mm(self, mat2):
    """aten::mm(Tensor self, Tensor mat2) -> Tensor"""
    assert self.dim() == 2 and mat2.dim() == 2 and self.shape[1] == mat2.shape[0] and self.dtype == mat2.dtype
    out = torch.empty((self.shape[0], mat2.shape[1]), dtype=self.dtype, device=self.device)
    return _mm_into(out, self, mat2, 1.0, 0.0)


def addmm(self, mat1, mat2, *, beta=1, alpha=1):
    """aten::addmm(Tensor self, Tensor mat1, Tensor mat2, *, Scalar beta=1, Scalar alpha=1) -> Tensor"""
    assert mat1.dim() == 2 and mat2.dim() == 2 and mat1.shape[1] == mat2.shape[0] and mat1.dtype == mat2.dtype
    m, n = mat1.shape[0], mat2.shape[1]
    if beta == 0:
        out = torch.empty((m, n), dtype=mat1.dtype, device=mat1.device)  # self is not read, NaNs included
    else:
        out = self.to(mat1.dtype).expand(m, n).clone(memory_format=torch.contiguous_format)
    return _mm_into(out, mat1, mat2, alpha, beta)


_offs_cache = {}


def _equal_offsets(device, batch, rows):
    """int32 device tensor [rows, 2 * rows, ..., batch * rows] (cached: it only depends on the shape)."""
    key = (device, batch, rows)
    t = _offs_cache.get(key)
    if t is None:
        if len(_offs_cache) > 256:
            _offs_cache.clear()
        t = (torch.arange(1, batch + 1, device=device, dtype=torch.int64) * rows).to(torch.int32)
        _offs_cache[key] = t
    return t


def bmm(self, mat2):
    """aten::bmm(Tensor self, Tensor mat2) -> Tensor.

    Tensor-core types run as ONE grouped launch: the batch is a grouped matmul over equal row segments of
    ``self`` viewed as ``[batch * m, k]`` (``group_mm``).  IEEE fp32, unaligned rows and tiny batches run
    one GEMM per batch entry."""
    assert self.dim() == 3 and mat2.dim() == 3 and self.shape[0] == mat2.shape[0] and self.shape[2] == mat2.shape[1]
    assert self.dtype == mat2.dtype
    batch, m, k = self.shape
    n = mat2.shape[2]
    code = _lib.FB_F32 if self.dtype in _EX_CODES else _code(self.dtype)  # (double / complex: one GEMM per entry)
    esz = self.element_size()
    if (batch >= 3 and code != _lib.FB_F32 and m > 0 and n > 0 and k > 0 and (k * esz) % 16 == 0 and (n * esz) % 16 == 0):
        from .ops.level3.group_gemm import group_mm

        a2 = self.reshape(batch * m, k)
        b3 = mat2 if (mat2.stride(2) == 1 or mat2.stride(1) == 1) else mat2.contiguous()
        ok = a2.data_ptr() % 16 == 0 and b3.data_ptr() % 16 == 0 and (b3.stride(0) * esz) % 16 == 0 and \
            (max(b3.stride(1), b3.stride(2)) * esz) % 16 == 0
        if ok:
            return group_mm(a2.contiguous(), b3, _equal_offsets(self.device, batch, m)).view(batch, m, n)
    out = torch.empty((batch, m, n), dtype=self.dtype, device=self.device)
    for i in range(batch):
        _mm_into(out[i], self[i], mat2[i], 1.0, 0.0)
    return out


def _grouped_mm(self, mat2, offs=None, bias=None, out_dtype=None):
    """aten::_grouped_mm(Tensor self, Tensor mat2, Tensor? offs, Tensor? bias, ScalarType? out_dtype) -> Tensor:
    the 2-D x 3-D form (row segments of ``self`` ending at ``offs`` times ``mat2[g]``) and the 3-D x 3-D form."""
    if bias is not None or (out_dtype is not None and out_dtype != self.dtype):
        raise NotImplementedError("flag_blas _grouped_mm: bias and out_dtype conversions are not provided")
    if self.dim() == 3 and mat2.dim() == 3 and offs is None:
        return bmm(self, mat2)
    if self.dim() == 2 and mat2.dim() == 3 and offs is not None:
        from .ops.level3.group_gemm import group_mm

        return group_mm(self, mat2, offs)
    raise NotImplementedError("flag_blas _grouped_mm: only [M, K] x [G, K, N] with row offsets and [B, M, K] x [B, K, N]")


def _mv_into(out, a, x, alpha, beta):
    m, n = a.shape
    if m == 0:
        return out
    if n == 0:
        return out.zero_() if beta == 0 else out.mul_(beta)
    if out.dtype in _EX_CODES:
        _mm_into_ex(out.view(m, 1), a, x.contiguous().view(n, 1), alpha, beta)
        return out
    a, trans, lda = as_operand(a)
    if x.stride(0) < 1:
        x = x.contiguous()
    code = _lib.FB_F32 if a.dtype == torch.float32 else _code(a.dtype)
    # the stored matrix is [m, lda] (trans = N) or [n, lda] (trans = T, product with its transpose)
    sm, sn = (m, n) if trans == CUBLAS_OP_N else (n, m)
    _gemv._call(code, "aten::mv", trans, sm, sn, float(alpha), a.data_ptr(), lda, x.data_ptr(), x.stride(0),
                float(beta), out.data_ptr(), 1, a.device)
    return out


def mv(self, vec):
    """aten::mv(Tensor self, Tensor vec) -> Tensor"""
    assert self.dim() == 2 and vec.dim() == 1 and self.shape[1] == vec.shape[0] and self.dtype == vec.dtype
    out = torch.empty((self.shape[0],), dtype=self.dtype, device=self.device)
    return _mv_into(out, self, vec, 1.0, 0.0)


def addmv(self, mat, vec, *, beta=1, alpha=1):
    """aten::addmv(Tensor self, Tensor mat, Tensor vec, *, Scalar beta=1, Scalar alpha=1) -> Tensor"""
    assert mat.dim() == 2 and vec.dim() == 1 and mat.shape[1] == vec.shape[0] and mat.dtype == vec.dtype
    if beta == 0:
        out = torch.empty((mat.shape[0],), dtype=mat.dtype, device=mat.device)
    else:
        out = self.to(mat.dtype).expand(mat.shape[0]).clone(memory_format=torch.contiguous_format)
    return _mv_into(out, mat, vec, alpha, beta)


# (aten key, function[, condition]) -- the reference's `_FULL_CONFIG` format.
_FULL_CONFIG = (
    ("mm", mm),
    ("addmm", addmm),
    ("bmm", bmm),
    ("mv", mv),
    ("addmv", addmv),
    ("_grouped_mm", _grouped_mm, lambda: hasattr(torch.ops.aten, "_grouped_mm")),
)
FULL_CONFIG_BY_FUNC = {}
for _item in _FULL_CONFIG:
    FULL_CONFIG_BY_FUNC.setdefault(_item[1].__name__, []).append(_item)


class Register:
    """Registers the selected table entries into a ``torch.library.Library`` under the CUDA key."""

    reg_key = "CUDA"

    def __init__(self, config, user_include_ops=None, user_exclude_ops=None, cpp_patched_ops=None, lib=None,
                 full_config_by_func=None):
        self.lib = lib
        self.all_ops = []
        self.all_keys = []
        include = list(user_include_ops or [])
        self.exclude_ops = [] if include else list(user_exclude_ops or [])
        patched = set(cpp_patched_ops or [])
        self.config = []
        for item in config:
            key, fn = item[0], item[1]
            if len(item) > 2 and not item[2]():
                continue
            if include:
                if fn.__name__ not in include and key not in include:
                    continue
            elif fn.__name__ in self.exclude_ops or key in self.exclude_ops or key in patched:
                continue
            self.config.append((key, fn))
        if include and not self.config:
            warnings.warn("only_enable failed: No op to register. Check if include is correct.")
        for key, fn in self.config:
            self.register_impl(key, fn)

    def register_impl(self, key, fn):
        if self.lib is None:
            raise ValueError("Library instance is not provided.")
        self.lib.impl(key, fn, self.reg_key)
        self.all_ops.append(fn.__name__)
        self.all_keys.append(key)

    def get_all_ops(self):
        return self.all_ops

    def get_all_keys(self):
        return self.all_keys

    def get_unused_ops(self):
        return self.exclude_ops


registrar = Register
current_work_registrar = None
_aten_lib = None


def _default_lib():
    global _aten_lib
    if _aten_lib is None:
        _aten_lib = torch.library.Library("aten", "IMPL")
    return _aten_lib


def _names(setting):
    if setting is None or setting == "default":
        return []
    if isinstance(setting, str):
        import yaml

        with open(setting) as f:
            data = yaml.safe_load(f) or {}
        if isinstance(data, dict):
            data = data.get("exclude") or data.get("include") or []
        return list(data)
    return list(setting)


def enable(lib=None, unused=None, registrar=Register, record=False, once=False, path=None):
    """Register every operator of the table except the names in ``unused`` (list, or a YAML path with an
    ``exclude:`` list).  Registration lasts for the life of ``lib`` (default: a process-wide library)."""
    global current_work_registrar
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)  # torch warns that an existing CUDA kernel is overridden
        current_work_registrar = registrar(_FULL_CONFIG, user_include_ops=[], user_exclude_ops=_names(unused),
                                           cpp_patched_ops=[], lib=lib if lib is not None else _default_lib())


def only_enable(lib=None, include=None, registrar=Register, record=False, once=False, path=None):
    """Register only the named operators (function names or aten keys)."""
    names = _names(include)
    if not names:
        warnings.warn("only_enable failed: No include entries resolved from list or yaml.")
        return
    global current_work_registrar
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        current_work_registrar = registrar(_FULL_CONFIG, user_include_ops=names, user_exclude_ops=[],
                                           cpp_patched_ops=[], full_config_by_func=FULL_CONFIG_BY_FUNC,
                                           lib=lib if lib is not None else _default_lib())


class use_blas:
    """``with flag_blas.use_blas(): ...`` -- the overrides are active inside the block only.
    ``include`` has priority over ``exclude``, as in the reference."""

    def __init__(self, exclude=None, include=None, record=False, once=False, path=None):
        self.exclude = exclude if isinstance(exclude, (list, tuple, set, str)) else []
        self.include = include if isinstance(include, (list, tuple, set, str)) else []
        self.lib = None

    def __enter__(self):
        self.lib = torch.library.Library("aten", "IMPL")
        if self.include:
            only_enable(lib=self.lib, include=self.include)
        else:
            enable(lib=self.lib, unused=self.exclude)
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        global current_work_registrar
        self.lib._destroy()
        self.lib = None
        current_work_registrar = None
        return False


def all_registered_ops():
    return current_work_registrar.get_all_ops() if current_work_registrar else []


def all_registered_keys():
    return current_work_registrar.get_all_keys() if current_work_registrar else []
