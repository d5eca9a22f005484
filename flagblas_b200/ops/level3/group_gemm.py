"""Grouped GEMM operators: ``group_bfgemm``, ``group_hgemm``, ``group_tf32gemm``,
``group_mm`` and the convenience wrapper ``group_gemm``.

Signatures follow the reference (``src/flag_blas/ops/level3/group_gemm.py:221-262``,
``:380-421``, ``:540-581``, ``:689-717``): every pointer / size / stride array is a
*device* tensor that is never read on the host; ``alpha`` / ``beta`` are shared by
all groups; the result is written through ``d_output_ptrs`` and ``group_out`` is
returned.  ``group_tf32gemm`` expects each ``B_g`` stored ``[n_g, k_g]``
(``group_gemm.py:488-504``), the 16-bit flavours ``[k_g, n_g]``.

``group_gemm(group_A, group_B, group_C, offs_table, alpha=, beta=)`` is the
signature the reference's ``tests/test_group_gemm.py:60-119`` calls but the
reference never defines; it is provided here on top of the grouped kernels.
"""
import torch

from ... import _lib

_cop = _lib.cop


def _group(code, b_k_contig, name, group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes,
           d_k_sizes, d_ldas, d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m=False):
    if use_small_m:
        # the caller's promise that no group has more than 64 rows: the library takes its small-M plan when the row
        # hint says so (any m_g is still computed correctly)
        M = min(int(M), 64 * int(group_size)) if int(M) > 0 else 64 * int(group_size)
    alpha = alpha.item() if isinstance(alpha, torch.Tensor) else float(alpha)
    beta = beta.item() if isinstance(beta, torch.Tensor) else float(beta)
    if group_size == 0:
        return group_out
    for t in (d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs):
        assert t.dtype == torch.int64 and t.is_cuda and t.is_contiguous() and t.numel() >= group_size
    for t in (d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs):
        assert t.dtype == torch.int32 and t.is_cuda and t.is_contiguous() and t.numel() >= group_size
    dev = d_a_ptrs.device
    stream, prev = _lib.enter(dev)
    try:
        # tile table + per-group tensor maps live in per-stream scratch
        nbytes = _cop.group_workspace_bytes(group_size)
        ws_ptr = _lib.scratch(dev, stream, nbytes)
        status = _cop.group_gemm(code, b_k_contig, d_a_ptrs.data_ptr(), d_b_ptrs.data_ptr(), d_c_ptrs.data_ptr(),
                                 d_output_ptrs.data_ptr(), d_m_sizes.data_ptr(), d_n_sizes.data_ptr(),
                                 d_k_sizes.data_ptr(), d_ldas.data_ptr(), d_ldbs.data_ptr(), d_ldcs.data_ptr(),
                                 group_size, int(M), int(N), int(K), alpha, beta, ws_ptr, nbytes, stream)
    finally:
        _lib.leave(prev)
    _lib.check(status, name)
    return group_out


def group_bfgemm(group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes, d_k_sizes, d_ldas,
                 d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m=False):
    """bf16 grouped GEMM (reference: ops/level3/group_gemm.py:221-262).

    ``use_small_m`` is the caller's promise that no group has more than 64 rows (the reference routes such calls
    to dedicated kernels, runtime/backend/_nvidia/hopper/ops/group_gemm.py:717-721); here it selects the small-M
    tile plan (tiles of up to 64 rows computed transposed, a deeper operand ring), which is also chosen by itself
    when ``M <= 64 * group_size``.  Results do not depend on it.
    """
    return _group(_lib.FB_BF16, 0, "group_bfgemm", group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs,
                  d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m)


def group_hgemm(group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes, d_k_sizes, d_ldas,
                d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m=False):
    """fp16 grouped GEMM (reference: ops/level3/group_gemm.py:380-421)."""
    return _group(_lib.FB_F16, 0, "group_hgemm", group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs,
                  d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m)


def group_tf32gemm(group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes, d_k_sizes, d_ldas,
                   d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m=False):
    """fp32-storage / TF32 grouped GEMM, B_g stored [n_g, k_g] (reference: group_gemm.py:540-581)."""
    return _group(_lib.FB_TF32, 1, "group_tf32gemm", group_out, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs,
                  d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs, group_size, M, N, K, alpha, beta, use_small_m)


class GroupPlan:
    """A grouped GEMM whose tile table and tensor maps are built once and reused by several runs
    (``fb_group_gemm_prepare`` / ``fb_group_gemm_run``; the reference has no such split, its kernels rebuild
    their per-group descriptors on every call).  Made by :func:`group_prepare`; ``run`` computes
    ``out_g = alpha * A_g @ B_g + beta * C_g`` with the addresses, sizes and pitches the arrays held at
    preparation time.  The plan owns its workspace and keeps the argument tensors alive."""

    def __init__(self, code, b_k_contig, name, arrays, group_size, M, N, K):
        self.code, self.b_k_contig, self.name = code, b_k_contig, name
        self.arrays, self.group_size, self.hints = arrays, int(group_size), (int(M), int(N), int(K))
        self.device = arrays[0].device
        self.workspace = None
        if self.group_size:
            nbytes = _cop.group_workspace_bytes(self.group_size)
            self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            stream, prev = _lib.enter(self.device)
            try:
                status = _cop.group_gemm_prepare(code, b_k_contig, *[t.data_ptr() for t in arrays], self.group_size,
                                                 *self.hints, self.workspace.data_ptr(), nbytes, stream)
            finally:
                _lib.leave(prev)
            _lib.check(status, name + " (prepare)")

    def run(self, group_out, alpha, beta):
        alpha = alpha.item() if isinstance(alpha, torch.Tensor) else float(alpha)
        beta = beta.item() if isinstance(beta, torch.Tensor) else float(beta)
        if self.group_size:
            stream, prev = _lib.enter(self.device)
            try:
                status = _cop.group_gemm_run(self.code, self.b_k_contig, self.group_size, *self.hints, alpha, beta,
                                             self.workspace.data_ptr(), self.workspace.numel(), stream)
            finally:
                _lib.leave(prev)
            _lib.check(status, self.name)
        return group_out


_PLAN_KINDS = {"group_bfgemm": (_lib.FB_BF16, 0), "group_hgemm": (_lib.FB_F16, 0), "group_tf32gemm": (_lib.FB_TF32, 1)}


def group_prepare(name, d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs,
                  d_ldcs, group_size, M, N, K, use_small_m=False) -> GroupPlan:
    """Build the device-side tables of ``name`` (``"group_bfgemm"``, ``"group_hgemm"`` or ``"group_tf32gemm"``) for
    these argument arrays once; ``plan.run(group_out, alpha, beta)`` then only launches the GEMM kernel."""
    code, b_k_contig = _PLAN_KINDS[name]
    for t in (d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs):
        assert t.dtype == torch.int64 and t.is_cuda and t.is_contiguous() and t.numel() >= group_size
    for t in (d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs):
        assert t.dtype == torch.int32 and t.is_cuda and t.is_contiguous() and t.numel() >= group_size
    if use_small_m:
        M = min(int(M), 64 * int(group_size)) if int(M) > 0 else 64 * int(group_size)
    arrays = (d_a_ptrs, d_b_ptrs, d_c_ptrs, d_output_ptrs, d_m_sizes, d_n_sizes, d_k_sizes, d_ldas, d_ldbs, d_ldcs)
    return GroupPlan(code, b_k_contig, name, arrays, group_size, M, N, K)


# fp32 tensors run with TF32 tensor-core products (fp32 accumulate, rtol 1e-3): an extension -- the reference's group_mm
# kernel forms fp32 products in IEEE fp32 (tl.dot(..., allow_tf32=False), ops/level3/group_gemm.py:656)
_CODES = {torch.bfloat16: _lib.FB_BF16, torch.float16: _lib.FB_F16, torch.float32: _lib.FB_TF32}


def group_mm(A: torch.Tensor, B: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """``C[o_{g-1}:o_g] = A[o_{g-1}:o_g] @ B[g]`` (reference: ops/level3/group_gemm.py:689-717).

    ``offs`` holds int32 cumulative end rows on the device.  Rows of ``C`` beyond
    ``offs[-1]`` are left uninitialised, as in the reference (``new_empty``).
    """
    assert A.dim() == 2
    assert B.dim() == 3
    M, K = A.shape
    num_groups, BK, N = B.shape
    assert num_groups == offs.numel()
    assert BK == K
    assert A.dtype == B.dtype and A.dtype in _CODES
    assert A.is_cuda and B.is_cuda and offs.is_cuda
    if A.stride(1) != 1:
        A = A.contiguous()
    if B.stride(2) == 1:
        b_k_contig, ldb = 0, B.stride(1)
    elif B.stride(1) == 1:
        b_k_contig, ldb = 1, B.stride(2)
    else:
        B = B.contiguous()
        b_k_contig, ldb = 0, B.stride(1)
    if offs.dtype != torch.int32:
        offs = offs.to(torch.int32)
    offs = offs.contiguous()
    C = A.new_empty(M, N)
    if M == 0 or N == 0 or num_groups == 0:
        return C
    stream, prev = _lib.enter(A.device)
    try:
        nbytes = _cop.group_workspace_bytes(num_groups)
        ws_ptr = _lib.scratch(A.device, stream, nbytes)
        status = _cop.group_mm(_CODES[A.dtype], b_k_contig, A.data_ptr(), A.stride(0), B.data_ptr(), ldb,
                               B.stride(0), C.data_ptr(), C.stride(0), offs.data_ptr(), num_groups, N, K,
                               ws_ptr, nbytes, stream)
    finally:
        _lib.leave(prev)
    _lib.check(status, "group_mm")
    return C


def group_gemm(group_A, group_B, group_C, offs_table, alpha=1.0, beta=0.0):
    """``out_g = alpha * A_g @ B_g + beta * C_g`` over row segments (bf16 / fp16; fp32 tensors run with TF32
    products, ``B_g`` stored ``[k, n]`` like the 16-bit types).

    ``offs_table[g] = [m_g, n, k, start_M, start_K, start_C]`` (a host list, as in
    the reference's ``tests/test_group_gemm.py:60-69``): ``A_g`` = ``m_g`` rows of
    ``group_A [sum m, k]`` from row ``start_M``, ``B_g`` = ``k`` rows of
    ``group_B [E*k, n]`` from row ``start_K``, ``C_g`` / ``out_g`` = ``m_g`` rows from
    row ``start_C``.  Returns a new tensor shaped like ``group_C``.
    """
    assert group_A.dtype == group_B.dtype == group_C.dtype and group_A.dtype in _CODES
    assert group_A.is_contiguous() and group_B.is_contiguous() and group_C.is_contiguous()
    dev = group_A.device
    out = torch.empty_like(group_C)
    G = len(offs_table)
    if G == 0:
        return out
    esz = group_A.element_size()
    lda, ldb, ldc = group_A.shape[1], group_B.shape[1], group_C.shape[1]
    rows = [[int(v) for v in r] for r in offs_table]
    ptrs = torch.tensor(
        [[group_A.data_ptr() + r[3] * lda * esz for r in rows],
         [group_B.data_ptr() + r[4] * ldb * esz for r in rows],
         [group_C.data_ptr() + r[5] * ldc * esz for r in rows],
         [out.data_ptr() + r[5] * ldc * esz for r in rows]], dtype=torch.int64).to(dev)
    sizes = torch.tensor(
        [[r[0] for r in rows], [r[1] for r in rows], [r[2] for r in rows],
         [lda] * G, [ldb] * G, [ldc] * G], dtype=torch.int32).to(dev)
    _group(_CODES[group_A.dtype], 0, "group_gemm", out, ptrs[0], ptrs[1], ptrs[2], ptrs[3], sizes[0], sizes[1], sizes[2],
           sizes[3], sizes[4], sizes[5], G, sum(r[0] for r in rows), rows[0][1], rows[0][2], alpha, beta)
    return out
