"""GEMM on operands that live in (pinned) host memory: copies and kernels overlapped on CUDA streams.

``gemm_from_host`` is the end-to-end form of the dense operators: A, B (and C when ``beta != 0``) start in
host memory, the result ends in host memory.  Doing that as copy-in, compute, copy-out in sequence leaves
the GPU idle for ~90 % of the time at PCIe speeds, so when op(A) is stored row-major (``transa = N``) the
call is cut into row blocks of A and C:

    stream "in"  : B -> device | A_0 [C_0] -> device | A_1 [C_1] -> device | ...
    stream "run" :                       wait A_0: C_0 = op   | wait A_1: C_1 = op | ...
    stream "out" :                                     wait C_0: C_0 -> host | ...

Host-to-device and device-to-host copies run at the same time (the link is full duplex) and every kernel
hides behind the copy of the next block, so a step costs about the time of the input copies alone.
Other layouts (``transa = T``: a row block of op(A) is a strided column block of the stored matrix) run the
three phases one after the other.

The kernels are the ordinary operators (``flagblas_b200.hgemm`` ...), called on row-block views.
"""
import torch

from . import ops
from .ops._constants import CUBLAS_OP_N

_streams = {}


def _get_streams(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _streams:
        _streams[key] = tuple(torch.cuda.Stream(device=device) for _ in range(4))
    return _streams[key]


def gemm_from_host(name, transa, transb, m, n, k, alpha, hA, lda, hB, ldb, beta, hC, ldc, dA, dB, dC, chunks=8):
    """``hC <- alpha * op(hA) * op(hB) + beta * hC`` through the device buffers ``dA, dB, dC``.

    ``name`` is a dense operator name (``"hgemm"``, ``"bfgemm"``, ``"tf32gemm"``, ``"sgemm"``); ``hA, hB, hC`` are
    host tensors (pinned memory makes the copies asynchronous) laid out exactly like the operator's
    arguments, ``dA, dB, dC`` device tensors of the same shapes.  Returns after the work is *enqueued*;
    the caller's current stream waits for the last copy-out, so ``torch.cuda.current_stream().synchronize()``
    (or any later work on that stream) sees the finished ``hC``.
    """
    op = getattr(ops, name)
    cur = torch.cuda.current_stream(dA.device)
    if transa != CUBLAS_OP_N or m < 2 * chunks or chunks <= 1:
        dA.copy_(hA, non_blocking=True)
        dB.copy_(hB, non_blocking=True)
        if beta != 0:
            dC.copy_(hC, non_blocking=True)
        op(transa, transb, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc)
        hC.copy_(dC, non_blocking=True)
        return
    s_in, s_run, s_out, _ = _get_streams(dA.device)
    for s in (s_in, s_run, s_out):
        s.wait_stream(cur)   # earlier work of the caller on these buffers comes first
    a2, c2, ha2, hc2 = dA.view(-1)[: m * lda].view(m, lda), dC.view(-1)[: m * ldc].view(m, ldc), \
        hA.view(-1)[: m * lda].view(m, lda), hC.view(-1)[: m * ldc].view(m, ldc)
    with torch.cuda.stream(s_in):
        dB.copy_(hB, non_blocking=True)
    step = -(-m // chunks)
    step = -(-step // 256) * 256  # whole 256-row tiles per block
    for r0 in range(0, m, step):
        r1 = min(m, r0 + step)
        with torch.cuda.stream(s_in):
            a2[r0:r1].copy_(ha2[r0:r1], non_blocking=True)
            if beta != 0:
                c2[r0:r1].copy_(hc2[r0:r1], non_blocking=True)
            ready = s_in.record_event()
        with torch.cuda.stream(s_run):
            s_run.wait_event(ready)
            op(transa, transb, r1 - r0, n, k, alpha, a2[r0:r1], lda, dB, ldb, beta, c2[r0:r1], ldc)
            done = s_run.record_event()
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            hc2[r0:r1].copy_(c2[r0:r1], non_blocking=True)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    cur.wait_stream(s_run)


def gemm_from_host_sharded(name, transa, transb, m, n_local, k, alpha, hA, lda, hB, ldb, beta, hC, ldc, dA, dB, dC, rank,
                           world, group=None, chunks=None, gather_stream=True):
    """:func:`gemm_from_host` for one process per GPU with the columns of ``C`` (and of ``B``) sharded over ``world``
    ranks: ``hB, hC, dB, dC`` are this rank's column shard (``n_local`` columns, densely pitched), ``hA`` / ``dA`` the
    whole ``A``, which every rank needs.

    Copying all of ``A`` from the host on every rank would move ``world`` times its size over the host's links each
    step.  Instead every rank copies a ``1 / world`` slice of each row block of ``A`` from its host memory and the ranks
    complete the block with one NCCL all-gather over NVLink (in place: a rank's slice is already where the gathered
    block wants it) on a stream of its own, so that the host link carries the next slice meanwhile; the GEMM of a
    block starts when its gather is done, copies out overlap as in the unsharded form.
    Collective: every rank of ``group`` must make the call with the same ``m, k, chunks``.

    ``chunks`` defaults to 8 row blocks for two ranks and 4 for more (measured on four B200s, fp16 8192^3: 3.39 / 3.31 /
    3.55 ms with 2 / 4 / 8 blocks; with the gathers queued behind the copies on one stream, ``gather_stream=False``,
    3.66 / 3.65 / 3.81 ms).  The step is bound by the host's links: four ranks copying at once reach 38 GB/s each.
    """
    import torch.distributed as tdist

    if chunks is None:
        chunks = 8 if world <= 2 else 4
    if world == 1:
        return gemm_from_host(name, transa, transb, m, n_local, k, alpha, hA, lda, hB, ldb, beta, hC, ldc, dA, dB, dC, chunks)
    op = getattr(ops, name)
    cur = torch.cuda.current_stream(dA.device)
    step = -(-m // max(chunks, 1))
    step = -(-step // (256 * world)) * (256 * world)  # whole tiles per block, whole rows per rank
    if transa != CUBLAS_OP_N or lda != k or m % world != 0 or step > m:
        # no contiguous row blocks to deal out: every rank fetches what it needs itself
        if n_local > 0:
            gemm_from_host(name, transa, transb, m, n_local, k, alpha, hA, lda, hB, ldb, beta, hC, ldc, dA, dB, dC, chunks)
        return
    s_in, s_run, s_out, s_gather = _get_streams(dA.device)
    if not gather_stream:
        s_gather = s_in  # the gathers queue behind the copies, on the same stream
    for s in (s_in, s_run, s_out, s_gather):
        s.wait_stream(cur)
    a2, ha2 = dA.view(-1)[: m * lda].view(m, lda), hA.view(-1)[: m * lda].view(m, lda)
    if n_local > 0:
        c2, hc2 = dC.view(-1)[: m * ldc].view(m, ldc), hC.view(-1)[: m * ldc].view(m, ldc)
    b_ready = None
    for r0 in range(0, m, step):
        r1 = min(m, r0 + step)
        rows = r1 - r0
        dealt = rows % world == 0
        # stream "in": nothing but host-to-device copies, back to back, so the link never waits for a collective
        with torch.cuda.stream(s_in):
            if dealt:
                sub = rows // world
                mine = a2[r0 + rank * sub: r0 + (rank + 1) * sub]
                mine.copy_(ha2[r0 + rank * sub: r0 + (rank + 1) * sub], non_blocking=True)
            else:
                a2[r0:r1].copy_(ha2[r0:r1], non_blocking=True)
            if beta != 0 and n_local > 0:
                c2[r0:r1].copy_(hc2[r0:r1], non_blocking=True)
            ready = s_in.record_event()
            if b_ready is None:
                # B follows the first slice of A: the first all-gather runs while B is on its way
                if n_local > 0:
                    dB.copy_(hB, non_blocking=True)
                b_ready = s_in.record_event()
        if dealt:
            # stream "gather": the ranks complete the block over NVLink while the next slice is copied in
            with torch.cuda.stream(s_gather):
                s_gather.wait_event(ready)
                tdist.all_gather_into_tensor(a2[r0:r1], mine, group=group)
                ready = s_gather.record_event()
        if n_local > 0:
            with torch.cuda.stream(s_run):
                s_run.wait_event(ready)
                s_run.wait_event(b_ready)
                op(transa, transb, rows, n_local, k, alpha, a2[r0:r1], lda, dB, ldb, beta, c2[r0:r1], ldc)
                done = s_run.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hc2[r0:r1].copy_(c2[r0:r1], non_blocking=True)
    for s in (s_out, s_in, s_run, s_gather):
        cur.wait_stream(s)
