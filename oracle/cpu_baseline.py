"""CPU timing leg for the benchmark: the GEMM hot path on the host's cores.  TEST/BENCH INFRASTRUCTURE ONLY.

The reference itself has no CPU implementation of this path other than Triton's
interpreter (seconds for a 512^3 problem), so the CPU baseline the task names is
``torch.matmul`` in fp32 on all host cores: 16-bit and TF32 inputs are upcast,
because CPU half-precision GEMM is not representative.  Only ``bench.py`` calls this.
"""
import os
import time

import torch


def host_threads():
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    return max(1, n)


def time_dense_rows(m, n, k, ta, tb, target_seconds=12.0, seed=1, scale=0.05, repeats=1):
    """Time ``C[:rows] = op(A)[:rows] @ op(B)`` in fp32 for a row sample sized to ~target_seconds.

    Returns (tflops, rows, total seconds timed, threads).  The inputs have the workload's shape and
    distribution; only the number of output rows is reduced.
    """
    threads = host_threads()
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    B = torch.randn((n, k) if tb else (k, n), generator=g) * scale
    opB = B.t() if tb else B
    probe_rows = min(m, 256)
    A = torch.randn((k, probe_rows) if ta else (probe_rows, k), generator=g) * scale
    opA = A.t() if ta else A
    torch.matmul(opA, opB)  # warm-up (thread pool, pages)
    t0 = time.perf_counter()
    torch.matmul(opA, opB)
    dt = max(time.perf_counter() - t0, 1e-6)
    rows = int(min(m, max(probe_rows, probe_rows * target_seconds / dt)))
    rows = max(64, rows // 64 * 64) if rows >= 64 else rows
    A = torch.randn((k, rows) if ta else (rows, k), generator=g) * scale
    opA = A.t() if ta else A
    # Repeat the sample until about target_seconds of CPU work has been timed (fast hosts finish
    # the whole workload in well under a second); report the mean.
    total, runs = 0.0, 0
    while runs < max(1, repeats) or (total < target_seconds and runs < 200):
        t0 = time.perf_counter()
        torch.matmul(opA, opB)
        total += time.perf_counter() - t0
        runs += 1
    mean = total / runs
    return 2.0 * rows * n * k / mean / 1e12, rows, total, threads
