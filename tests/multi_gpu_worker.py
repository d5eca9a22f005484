"""One rank of the multi-GPU checks (launched by tests/test_multi_gpu.py through torch.distributed.run).

Every rank builds the same seeded operands, runs its share through the sharded entry points and compares what it
ends up with against the single-GPU operator on the same inputs.  Prints ``rank R ok`` or raises."""
import os
import sys

import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import flagblas_b200 as fb  # noqa: E402
from flagblas_b200 import dist as fbdist, host as fbhost  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    tdist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device="cpu").manual_seed(7)
    m, n, k = 2048 * world, 1536, 1024  # (row blocks that split evenly over the ranks; a ragged last column shard)
    A = (torch.randn(m, k, generator=g) * 0.25).half()
    B = (torch.randn(k, n, generator=g) * 0.25).half()
    C0 = torch.randn(m, n, generator=g).half()
    Ad, Bd = A.to(dev), B.to(dev)
    want = C0.to(dev)
    fb.hgemm(0, 0, m, n, k, 1.5, Ad, k, Bd, n, 0.5, want, n)

    # 1. strided column shard of full-size operands, then the all-gather of the columns
    C = C0.to(dev)
    n0, n1 = fbdist.sharded_gemm("hgemm", 0, 0, m, n, k, 1.5, Ad, k, Bd, n, 0.5, C, n, rank, world)
    assert torch.equal(C[:, n0:n1], want[:, n0:n1]), "column shard differs from the single-GPU result"
    if n0 > 0:
        assert torch.equal(C[:, :n0], C0.to(dev)[:, :n0]), "a rank wrote outside its columns"
    fbdist.all_gather_columns(C, m, n, n, rank, world)
    assert torch.equal(C, want), "gathered C differs"

    # 2. the same by row blocks with the exchange on a side stream
    C = C0.to(dev)
    fbdist.sharded_gemm_gather("hgemm", 0, 0, m, n, k, 1.5, Ad, k, Bd, n, 0.5, C, n, rank, world)
    torch.cuda.synchronize()
    torch.testing.assert_close(C.float(), want.float(), rtol=2e-3, atol=2e-3)

    # 3. operands in pinned host memory: 1 / world of every row block of A per rank, completed over NVLink
    nl = n1 - n0
    hA, hB = A.pin_memory(), B[:, n0:n1].contiguous().pin_memory()
    hC = C0[:, n0:n1].contiguous().pin_memory()
    dA = torch.zeros(m, k, dtype=torch.float16, device=dev)
    dB = torch.empty(k, max(nl, 1), dtype=torch.float16, device=dev)[:, :nl]
    dC = torch.empty(m, max(nl, 1), dtype=torch.float16, device=dev)[:, :nl]
    for _ in range(2):  # (the second pass reuses the buffers: no stale event or stream state)
        hC.copy_(C0[:, n0:n1])
        fbhost.gemm_from_host_sharded("hgemm", 0, 0, m, nl, k, 1.5, hA, k, hB, nl, 0.5, hC, nl, dA, dB, dC, rank, world)
        torch.cuda.synchronize()
        assert torch.equal(dA, Ad), "A was not completed by the all-gather"
        torch.testing.assert_close(hC.float(), want[:, n0:n1].float().cpu(), rtol=2e-3, atol=2e-3)

    # 4. grouped GEMM dealt by FLOPs: every rank's pieces land in its copy of the output, the union is the whole
    E, K, N = 6, 512, 768
    ms = [300, 17, 1024, 0, 129, 640]
    T = sum(ms)
    X = (torch.randn(T, K, generator=g) * 0.25).bfloat16().to(dev)
    W = (torch.randn(E * K, N, generator=g) * 0.05).bfloat16().to(dev)
    full = torch.zeros(T, N, dtype=torch.bfloat16, device=dev)
    ap, bp, op_, s = [], [], [], 0
    for e, mg in enumerate(ms):
        ap.append(X.data_ptr() + s * K * 2); bp.append(W.data_ptr() + e * K * N * 2); op_.append(full.data_ptr() + s * N * 2)
        s += mg
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    fb.group_bfgemm(full, i64(ap), i64(bp), i64(op_), i64(op_), i32(ms), i32([N] * E), i32([K] * E), i32([K] * E),
                    i32([N] * E), i32([N] * E), E, T, N, K, 1.0, 0.0)
    mine = torch.zeros(T, N, dtype=torch.bfloat16, device=dev)
    shift = mine.data_ptr() - full.data_ptr()
    op_m = [p + shift for p in op_]
    pieces = fbdist.plan_group_shards(ms, [N] * E, [K] * E, world)
    arrs, count = fbdist.shard_group_arrays(pieces[rank], ap, bp, op_m, op_m, ms, [N] * E, [K] * E, [K] * E, [N] * E,
                                            [N] * E, 2, dev)
    if count:
        rows = sum(r for _, _, r in pieces[rank])
        fb.group_bfgemm(mine, *arrs, count, rows, N, K, 1.0, 0.0)
    torch.cuda.synchronize()
    tdist.all_reduce(mine)  # (ranks write disjoint rows of zeros-initialised copies: the sum is the union)
    torch.testing.assert_close(mine.float(), full.float(), rtol=1e-2, atol=1e-2)
    assert fb.device_status() == 0
    tdist.barrier()
    print("rank %d ok" % rank, flush=True)
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
