"""Multi-GPU execution of the GEMM path: one process per GPU, no data-path collective.

The reference has no multi-GPU code at all; this module adds the two natural
shardings of the path:

* a single large GEMM is split by columns of ``C`` (N-split): rank ``r`` owns a
  contiguous, tile-aligned column range, reads all of ``A`` and its slice of
  ``B`` and writes its slice of ``C`` in place -- output tiles are independent,
  so nothing is exchanged.  ``all_gather_columns`` optionally assembles the full
  ``C`` on every rank with one NCCL all-gather over NVLink;
* a grouped GEMM is split by FLOP-balanced assignment of groups to ranks
  (longest-processing-time first), cutting any group that alone exceeds a
  rank's fair share into row slices (``B_g`` is then used by several ranks).

Everything here is host logic over ``torch.distributed``; the arithmetic is the
same single-GPU operators.
"""
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .ops._constants import CUBLAS_OP_N


def column_ranges(n: int, world: int, align: int = 256) -> List[Tuple[int, int]]:
    """Split ``[0, n)`` into ``world`` contiguous ranges whose interior boundaries are
    multiples of ``align`` (the widest tile), as evenly as the alignment allows.
    Trailing ranks may get an empty range when ``n`` is small."""
    assert n >= 0 and world >= 1 and align >= 1
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        nb = base + (1 if r < extra else 0)
        end = min(n, start + nb * align)
        out.append((start, end))
        start = end
    return out


def sharded_gemm(name: str, transa: int, transb: int, m: int, n: int, k: int, alpha, A: torch.Tensor, lda: int,
                 B: torch.Tensor, ldb: int, beta, C: torch.Tensor, ldc: int, rank: int, world: int,
                 align: int = 256, launch: Optional[Callable] = None) -> Tuple[int, int]:
    """Run this rank's column shard of the dense operator ``name``
    (``"hgemm"`` / ``"bfgemm"`` / ``"tf32gemm"`` / ``"sgemm"``).

    ``A``, ``B``, ``C`` are full-size operands in this rank's memory (``A`` replicated; of ``B``
    and ``C`` only the rank's columns are touched), validated exactly like the single-GPU call.
    The shard is the same GEMM with ``n`` narrowed and the ``B`` / ``C`` base addresses advanced;
    leading dimensions are unchanged, so nothing is copied.  Returns the column range.

    ``launch`` replaces the native launch (same arguments as ``ops.level3.gemm._launch``); the
    CPU tests of the sharding logic use it, production code leaves it ``None``.
    """
    from .ops.level3 import gemm as _g

    code, dtype = _g.OPS[name]
    n0, n1 = column_ranges(n, world, align)[rank]
    if launch is None:
        _g._validate(dtype, name, transa, transb, m, n, k, A, lda, B, ldb, C, ldc)
    alpha = _g._scalar(alpha)
    beta = _g._scalar(beta)
    if m == 0 or n == 0 or n1 <= n0:
        return n0, n1
    _g._validate_extents(transa, transb, m, n, k, A, lda, B, ldb, C, ldc)
    esz = B.element_size()
    b_off = n0 if transb == CUBLAS_OP_N else n0 * ldb  # [k, ldb]: n0 columns in; [n, ldb]: n0 rows in
    fn = launch or _g._launch
    fn(code, name, transa, transb, m, n1 - n0, k, alpha, A.data_ptr(), lda, B.data_ptr() + b_off * esz, ldb, beta,
       C.data_ptr() + n0 * esz, ldc, A.device)
    return n0, n1


def all_gather_columns(C_local: torch.Tensor, m: int, n: int, ldc: int, rank: int, world: int, align: int = 256,
                       group=None) -> None:
    """Make ``C`` complete on every rank: one all-gather of the packed column shards,
    then each shard is copied into its columns of the local row-major ``C``."""
    import torch.distributed as dist

    ranges = column_ranges(n, world, align)
    width = max(e - s for s, e in ranges)
    c2d = C_local.view(-1)[: m * ldc].view(m, ldc)
    n0, n1 = ranges[rank]
    if n1 - n0 == width:
        packed = c2d[:, n0:n1].contiguous()
    else:  # a narrower (or empty) last shard travels zero-padded to the common width
        packed = torch.zeros(m, width, dtype=C_local.dtype, device=C_local.device)
        if n1 > n0:
            packed[:, : n1 - n0].copy_(c2d[:, n0:n1])
    flat = torch.empty(world * m, width, dtype=C_local.dtype, device=C_local.device)  # rank-major concatenation
    dist.all_gather_into_tensor(flat, packed, group=group)
    gathered = flat.view(world, m, width)
    for r, (s, e) in enumerate(ranges):
        if r != rank and e > s:
            c2d[:, s:e].copy_(gathered[r, :, : e - s])


_gather_streams = {}


def sharded_gemm_gather(name: str, transa: int, transb: int, m: int, n: int, k: int, alpha, A: torch.Tensor, lda: int,
                        B: torch.Tensor, ldb: int, beta, C: torch.Tensor, ldc: int, rank: int, world: int,
                        align: int = 256, chunks: int = 4, group=None, launch: Optional[Callable] = None) -> None:
    """:func:`sharded_gemm` followed by :func:`all_gather_columns`, by row blocks: the GEMM runs in row blocks of
    ``A`` / ``C`` on the current stream and every finished block is exchanged on a side stream while the next one
    computes.  Measured on two B200s (fp16 8192^3, 64 MiB per rank) this is SLOWER than the GEMM followed by one
    exchange (0.82 against 0.73 ms; the GEMM alone 0.40 ms): a quarter of the rows is 128 tiles on 74 CTA pairs, so
    every block pays the tile quantisation the whole shard avoids, the persistent GEMM occupies every SM and leaves
    the collective's kernels little room beside it, and the per-block packing and unpacking launches add up.  Kept
    for callers whose shards are large enough to amortise that; ``bench.py`` reports both.  ``A``, ``B``, ``C`` are full-size operands with their
    original leading dimensions (the rank's shard of ``C`` is a strided column block of the full ``C``); afterwards
    every rank holds the complete ``C``.  Needs ``transa = N`` to cut row blocks; other layouts run the two phases
    one after the other."""
    if world == 1 or transa != CUBLAS_OP_N or chunks <= 1 or m < 2 * chunks:
        sharded_gemm(name, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, rank, world, align, launch)
        if world > 1:
            all_gather_columns(C, m, n, ldc, rank, world, align, group)
        return
    a2 = A.view(-1)[: m * lda].view(m, lda)
    c2 = C.view(-1)[: m * ldc].view(m, ldc)
    step = -(-m // chunks)
    step = -(-step // 256) * 256  # whole 256-row tiles per block
    blocks = [(r0, min(m, r0 + step)) for r0 in range(0, m, step)]
    if not C.is_cuda:
        # host tensors (the CPU tests of the sharding logic): the same blocks, one after the other
        for r0, r1 in blocks:
            sharded_gemm(name, transa, transb, r1 - r0, n, k, alpha, a2[r0:r1], lda, B, ldb, beta, c2[r0:r1], ldc, rank,
                         world, align, launch)
            all_gather_columns(c2[r0:r1], r1 - r0, n, ldc, rank, world, align, group)
        return
    dev = C.device
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _gather_streams:
        _gather_streams[key] = torch.cuda.Stream(device=dev)
    side = _gather_streams[key]
    cur = torch.cuda.current_stream(dev)
    side.wait_stream(cur)
    for r0, r1 in blocks:
        sharded_gemm(name, transa, transb, r1 - r0, n, k, alpha, a2[r0:r1], lda, B, ldb, beta, c2[r0:r1], ldc, rank, world,
                     align, launch)
        done = cur.record_event()
        with torch.cuda.stream(side):
            side.wait_event(done)
            all_gather_columns(c2[r0:r1], r1 - r0, n, ldc, rank, world, align, group)
    cur.wait_stream(side)


def plan_group_shards(m_sizes: Sequence[int], n_sizes: Sequence[int], k_sizes: Sequence[int], world: int,
                      row_align: int = 128) -> List[List[Tuple[int, int, int]]]:
    """FLOP-balanced assignment of grouped-GEMM work to ranks.

    Returns, per rank, a list of ``(group, row_start, row_count)`` pieces.  Groups whose FLOPs
    exceed the per-rank fair share are first cut into row slices (multiples of ``row_align``
    rows) no larger than that share; pieces are then placed largest first on the least
    loaded rank (LPT).  Zero-row groups are dropped.
    """
    assert world >= 1
    flops = [2.0 * m * n * k for m, n, k in zip(m_sizes, n_sizes, k_sizes)]
    total = sum(flops)
    if total == 0:
        return [[] for _ in range(world)]
    share = total / world
    pieces = []  # (flops, group, row_start, rows)
    for g, (m, n, k) in enumerate(zip(m_sizes, n_sizes, k_sizes)):
        if m <= 0 or n <= 0:
            continue
        per_row = 2.0 * n * k
        if per_row == 0 or flops[g] <= share:
            pieces.append((flops[g], g, 0, m))
            continue
        max_rows = max(row_align, int(share / per_row) // row_align * row_align)
        start = 0
        while start < m:
            rows = min(max_rows, m - start)
            pieces.append((rows * per_row, g, start, rows))
            start += rows
    pieces.sort(key=lambda p: (-p[0], p[1], p[2]))
    load = [0.0] * world
    plan: List[List[Tuple[int, int, int]]] = [[] for _ in range(world)]
    for f, g, s, rws in pieces:
        r = min(range(world), key=lambda i: (load[i], i))
        plan[r].append((g, s, rws))
        load[r] += f
    for p in plan:
        p.sort()
    return plan


def plan_imbalance(plan, m_sizes, n_sizes, k_sizes) -> float:
    """max rank load / ideal load for a plan from :func:`plan_group_shards` (1.0 = perfect)."""
    loads = [sum(2.0 * rows * n_sizes[g] * k_sizes[g] for g, _, rows in p) for p in plan]
    total = sum(loads)
    return max(loads) / (total / len(plan)) if total else 1.0


def shard_group_arrays(pieces, a_ptrs, b_ptrs, c_ptrs, out_ptrs, m_sizes, n_sizes, k_sizes, ldas, ldbs, ldcs,
                       elem_size: int, device):
    """Device argument arrays of one rank's share of a grouped GEMM.

    ``pieces`` is one entry of :func:`plan_group_shards` -- ``(group, row_start, rows)`` triples; the
    other arguments are the *host* lists that describe the whole problem (addresses as ints).  A piece
    is the row slice ``[row_start, row_start + rows)`` of its group: A, C and out advance by
    ``row_start`` rows, B is shared.  Returns the eleven tensors ``group_bfgemm`` / ``group_hgemm`` /
    ``group_tf32gemm`` take after ``group_out`` (int64 addresses, int32 sizes and strides) and the
    piece count.
    """
    ap, bp, cp, op, ms, ns, ks, la, lb, lc = ([] for _ in range(10))
    for g, start, rows in pieces:
        ap.append(a_ptrs[g] + start * ldas[g] * elem_size)
        bp.append(b_ptrs[g])
        cp.append(c_ptrs[g] + start * ldcs[g] * elem_size)
        op.append(out_ptrs[g] + start * ldcs[g] * elem_size)
        ms.append(rows); ns.append(n_sizes[g]); ks.append(k_sizes[g])
        la.append(ldas[g]); lb.append(ldbs[g]); lc.append(ldcs[g])
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=device)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)  # noqa: E731
    return (i64(ap), i64(bp), i64(cp), i64(op), i32(ms), i32(ns), i32(ks), i32(la), i32(lb), i32(lc)), len(pieces)
