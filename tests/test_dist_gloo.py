"""Multi-process coverage of the N>1 path on CPU: two gloo ranks run the column-sharded GEMM and the
optional all-gather.  The native launch is replaced by a stand-in that performs the same memory
effect on host buffers with the CPU oracle (the sharding, pointer arithmetic and collective are the
code under test; the arithmetic is checked on the GPU elsewhere)."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as tdist
import torch.multiprocessing as mp

from flagblas_b200 import dist as fbdist
from oracle import gemm_oracle as go


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _host_launch(code, name, transa, transb, m, n, k, alpha, a_ptr, lda, b_ptr, ldb, beta, c_ptr, ldc, device):
    """Same contract as ops.level3.gemm._launch, on host memory: fp32 only."""
    def view(ptr, count):
        return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_float)), shape=(count,))

    a = view(a_ptr, (k if transa else m) * lda)
    # a column shard starts n0 elements into the matrix: only rows*ld - n0 elements lie behind the pointer
    b_rows = n if transb else k
    b = view(b_ptr, (b_rows - 1) * ldb + (k if transb else n))
    c = view(c_ptr, (m - 1) * ldc + n)
    bb = np.zeros(b_rows * ldb, dtype=np.float32); bb[: b.size] = b
    cc = np.zeros(m * ldc, dtype=np.float32); cc[: c.size] = c
    go.gemm("fp32", transa, transb, m, n, k, alpha, a, lda, bb, ldb, beta, cc, ldc)
    c[...] = cc[: c.size]


def _worker(rank, world, port, transb, gather, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    tdist.init_process_group("gloo", rank=rank, world_size=world)
    m, n, k = (96 if gather != "blocks" else 600), 600, 40   # 600 columns, 256-aligned boundaries -> shards [0,512) and [512,600)
    g = torch.Generator().manual_seed(7)
    A = torch.randn(m, k, generator=g)
    B = torch.randn((n, k) if transb else (k, n), generator=g)
    C0 = torch.randn(m, n, generator=g)
    C = C0.clone()
    ref = 1.5 * (A.double() @ (B.double().t() if transb else B.double())) + 0.5 * C0.double()
    if gather == "blocks":
        # GEMM by row blocks, each block's column shards exchanged as soon as it is done (three blocks of 256 rows here)
        fbdist.sharded_gemm_gather("sgemm", 0, transb, m, n, k, 1.5, A, k, B, B.shape[1], 0.5, C, n, rank, world, chunks=3,
                                   launch=_host_launch)
        ok = torch.allclose(C.double(), ref, rtol=1e-5, atol=1e-4)
        out_q.put((rank, fbdist.column_ranges(n, world)[rank], bool(ok)))
        tdist.barrier()
        tdist.destroy_process_group()
        return
    n0, n1 = fbdist.sharded_gemm("sgemm", 0, transb, m, n, k, 1.5, A, k, B, B.shape[1], 0.5, C, n, rank, world,
                                 launch=_host_launch)
    ok = torch.allclose(C[:, n0:n1].double(), ref[:, n0:n1], rtol=1e-5, atol=1e-4)
    # columns of the other rank are untouched
    mask = torch.ones(n, dtype=torch.bool); mask[n0:n1] = False
    ok = ok and torch.equal(C[:, mask], C0[:, mask])
    if gather:
        fbdist.all_gather_columns(C, m, n, n, rank, world)
        ok = ok and torch.allclose(C.double(), ref, rtol=1e-5, atol=1e-4)
    out_q.put((rank, (n0, n1), bool(ok)))
    tdist.barrier()
    tdist.destroy_process_group()


@pytest.mark.parametrize("transb,gather", [(0, False), (1, True), (0, True), (0, "blocks"), (1, "blocks")])
def test_two_ranks_column_shards(transb, gather):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, transb, gather, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [(0, 512), (512, 600)]
    assert all(r[2] for r in res)
