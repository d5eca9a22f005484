#!/usr/bin/env python
"""Benchmark of the GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  The headline workload is the large square fp16 GEMM:
``hgemm`` fp16, M=N=K=8192, NN, alpha=1, beta=0, A,B ~ N(0,1)*0.05 (seed 1), fp32
accumulate, fp16 output.  A "step" is one full GEMM.  With N > 1 GPUs the same GEMM is
column-sharded (N-split) across the ranks, one process per GPU, with no collective on the
data path (strong scaling: total work fixed).

``value``   : device-resident TFLOP/s (inputs in HBM, CUDA events, max over ranks).
``e2e``     : the same metric through the public host-memory entry (``flagblas_b200.host.gemm_from_host``):
              per step pinned-host -> device copies of A and B (and C when beta != 0), the GEMM, and the
              device -> host copy of C, overlapped on CUDA streams (row blocks of A / C) where the layout allows.
``roofline``: tensor-core roofline of the GEMM kernel (2*m*n*k FLOPs per launch / event time).
``cpu_baseline``: torch.matmul fp32 on the host cores over a bounded row sample (rank 0, N=1).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (operator, kind, transa, transb, m, n, k, alpha, beta, scaleA, scaleB, seed)
    "hgemm_8192_nn": ("hgemm", "fp16", 0, 0, 8192, 8192, 8192, 1.0, 0.0, 0.05, 0.05, 1),
    "bfgemm_mlp_nt": ("bfgemm", "bf16", 0, 1, 16384, 14336, 4096, 1.0, 1.0, 1.0, 0.02, 2),
    "tf32gemm_skinny_tn": ("tf32gemm", "tf32", 1, 0, 64, 16384, 16384, 1.5, 0.5, 0.577, 0.577, 4),
    "tf32gemm_8192_tn": ("tf32gemm", "tf32", 1, 0, 8192, 8192, 8192, 1.5, 0.5, 0.577, 0.577, 4),
    "tf32gemm_16384_tn": ("tf32gemm", "tf32", 1, 0, 16384, 16384, 16384, 1.5, 0.5, 0.577, 0.577, 4),
    # a decode step's shape: 64 tokens against a square weight matrix stored [n, k] (latency and HBM bound)
    "bfgemm_decode64_nt": ("bfgemm", "bf16", 0, 1, 64, 4096, 4096, 1.0, 0.0, 1.0, 0.02, 6),
    "sgemm_512_nn": ("sgemm", "fp32", 0, 0, 512, 512, 512, 1.0, 0.0, 0.577, 0.577, 0),
    "sgemm_4096_nn": ("sgemm", "fp32", 0, 0, 4096, 4096, 4096, 1.0, 0.0, 0.577, 0.577, 0),
}
# grouped MoE workload: 64 experts sharing K and N, token counts ~ Multinomial(T, Zipf(1.2)), seed 3
MOE = {"name": "group_bfgemm_moe64", "experts": 64, "k": 4096, "n": 1536, "tokens": 32768, "zipf": 1.2, "seed": 3}
HEADLINE = "hgemm_8192_nn"

_REAL_STDOUT = None


def claim_stdout():
    """Keep stdout for the one JSON line: whatever else writes to file descriptor 1 from here on (the NCCL
    version banner, library chatter) is sent to stderr instead."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line):
    out = _REAL_STDOUT if _REAL_STDOUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()
FALLBACK_TENSOR_PEAK = 1590.0  # TFLOP/s, earlier measurement on this pool, used only without MEASURED_PEAKS.json


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except (OSError, KeyError, ValueError):
        return FALLBACK_TENSOR_PEAK, "fallback"


def measured(key, fallback):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)[key]), "measured (MEASURED_PEAKS.json %s)" % key
    except (OSError, KeyError, ValueError):
        return fallback, "fallback"


def ncu_traffic(workload):
    """DRAM bytes per launch from the committed ncu summary, if one exists for this workload."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(workload)
    except (OSError, ValueError):
        return None


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML while a region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device_index, period=0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self._stop, self._thread, self.h = period, threading.Event(), None, None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = getattr(torch.cuda.get_device_properties(torch_device_index), "uuid", None)
            if uuid is not None:
                try:
                    self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
                except Exception:
                    self.h = None
            if self.h is None:
                vis = os.environ.get("CUDA_VISIBLE_DEVICES")
                idx = int(vis.split(",")[torch_device_index]) if vis and vis.split(",")[0].isdigit() else torch_device_index
                self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.h = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def _time(fn, torch, steps=10, warmup=3):
    # a short idle first: the previous workload may have left the GPU at its power limit, and a kernel that is
    # timed right behind it would be measured at the reduced clock of its predecessor
    torch.cuda.synchronize()
    time.sleep(0.5)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # calls of a few microseconds: ten of them end before the clocks have left their idle state and before the
    # launch queue holds more than one call, so such workloads run until about 2 ms have been timed (at most 400 calls)
    t0 = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    once = time.perf_counter() - t0
    steps = max(steps, min(400, int(2e-3 / max(once, 1e-6))))
    for _ in range(min(steps, 50)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _time_cold(fn, torch, dev, steps=10, warmup=3):
    """Mean time of single launches each of which finds L2 holding none of its operands: a buffer twice the size of
    L2 is rewritten before every launch (outside the timed interval)."""
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(steps):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / steps


def moe_setup(torch, dev, token_counts, K, N, seed):
    """Device tensors and the operator's argument tuple for a grouped bf16 GEMM over stacked token rows."""
    E, T = len(token_counts), sum(token_counts)
    g = torch.Generator(device=dev).manual_seed(seed)
    A = torch.randn(T, K, generator=g, device=dev).bfloat16()
    B = (torch.randn(E * K, N, generator=g, device=dev) * 0.02).bfloat16()
    O = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
    ap, bp, op_, s = [], [], [], 0
    for e, mg in enumerate(token_counts):
        ap.append(A.data_ptr() + s * K * 2); bp.append(B.data_ptr() + e * K * N * 2); op_.append(O.data_ptr() + s * N * 2); s += mg
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    args = (O, i64(ap), i64(bp), i64(op_), i64(op_), i32(token_counts), i32([N] * E), i32([K] * E), i32([K] * E),
            i32([N] * E), i32([N] * E), E, T, N, K, 1.0, 0.0)
    return (A, B, O), args


def other_configs(fb, torch, dev):
    """Short device-resident timings of the other benchmark workloads (not the headline)."""
    peak, _ = measured_peak()
    hbm, _ = measured("hbm_gbs", 6650.0)
    out = {}
    dts = {"fp16": torch.float16, "bf16": torch.bfloat16, "tf32": torch.float32, "fp32": torch.float32}
    for name, (op, kind, ta, tb, m, n, k, alpha, beta, sa, sb, seed) in WORKLOADS.items():
        if name == HEADLINE:
            continue
        g = torch.Generator(device=dev).manual_seed(seed)
        A = (torch.randn((k, m) if ta else (m, k), generator=g, device=dev) * sa).to(dts[kind])
        B = (torch.randn((n, k) if tb else (k, n), generator=g, device=dev) * sb).to(dts[kind])
        C = (torch.randn(m, n, generator=g, device=dev) * 0.02).to(dts[kind])
        fn = getattr(fb, op)
        ms = _time(lambda: fn(ta, tb, m, n, k, alpha, A, A.shape[1], B, B.shape[1], beta, C, n), torch)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        nbytes = A.element_size() * (m * k + k * n + m * n * (2 if beta != 0 else 1))
        rec = {"tflops": tf, "ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9}
        if name == "tf32gemm_skinny_tn":
            rec.update(bound="hbm", frac=rec["gbs"] / hbm, peak=hbm)
        elif name == "bfgemm_decode64_nt":
            # back to back its 32 MiB of weights stay in the 126 MB L2: the HBM roofline applies to launches that
            # find L2 cold, timed one by one with L2 rewritten in between
            cold = _time_cold(lambda: fn(ta, tb, m, n, k, alpha, A, A.shape[1], B, B.shape[1], beta, C, n), torch, dev)
            # context: cuBLAS (torch.matmul) on the same operands, timed the same two ways
            opB = B.t() if tb else B
            cublas_ms = _time(lambda: torch.matmul(A, opB, out=C), torch)
            cublas_cold = _time_cold(lambda: torch.matmul(A, opB, out=C), torch, dev)
            rec.update(bound="latency (operands L2-resident between back-to-back launches)", ms_l2_cold=cold,
                       gbs_l2_cold=nbytes / (cold * 1e-3) / 1e9, frac=nbytes / (cold * 1e-3) / 1e9 / hbm, peak=hbm,
                       frac_is="HBM roofline of the L2-cold launches", cublas_ms=cublas_ms, cublas_ms_l2_cold=cublas_cold)
        elif kind == "tf32":
            # no measured TF32 figure exists: the denominator is assumed, half the measured 16-bit rate; cuBLAS's
            # TF32 GEMM on the same operands is timed beside it as context
            torch.backends.cuda.matmul.allow_tf32 = True
            opA, opB = (A.t() if ta else A), (B.t() if tb else B)
            cms = _time(lambda: torch.matmul(opA, opB), torch, steps=5)
            torch.backends.cuda.matmul.allow_tf32 = False
            rec.update(bound="tensor", frac=tf / (peak / 2), peak=peak / 2,
                       peak_source="assumed: MEASURED_PEAKS.json bf16_tflops / 2 (no measured TF32 figure)",
                       cublas_tf32_tflops=2.0 * m * n * k / (cms * 1e-3) / 1e12)
        elif kind == "fp32":
            ffma_peak = 148 * 128 * 2 * 1.965e9 / 1e12   # SMs x FP32 lanes x 2 FLOP x max SM clock
            rec.update(bound="fp32 FFMA" + (" (latency bound at this size)" if m <= 512 else ""), frac=tf / ffma_peak,
                       peak=ffma_peak)
        else:
            rec.update(bound="tensor", frac=tf / peak, peak=peak)
        out[name] = rec
        del A, B, C
    # grouped MoE workload: 64 experts, K=4096, N=1536, Zipf(1.2) token counts, bf16
    E, K, N, T = MOE["experts"], MOE["k"], MOE["n"], MOE["tokens"]
    keep, args = moe_setup(torch, dev, moe_token_counts(torch), K, N, MOE["seed"])
    ms = _time(lambda: fb.group_bfgemm(*args), torch)
    tf = 2.0 * T * N * K / (ms * 1e-3) / 1e12
    out["group_bfgemm_moe64"] = {"tflops": tf, "ms": ms, "bound": "tensor", "frac": tf / peak, "peak": peak}
    # the same call with the tile table and tensor maps built once and reused (group_prepare / plan.run): what a caller
    # that runs one routing through several layers pays per call
    plan = fb.group_prepare("group_bfgemm", *args[1:15])
    ms = _time(lambda: plan.run(args[0], 1.0, 0.0), torch)
    tf = 2.0 * T * N * K / (ms * 1e-3) / 1e12
    out["group_bfgemm_moe64_prepared"] = {"tflops": tf, "ms": ms, "bound": "tensor", "frac": tf / peak, "peak": peak}
    del keep, args, plan
    # the same experts at decode time: at most 64 tokens each (the reference's small-M case).  Every expert's weights
    # are read once for a handful of rows, so HBM bounds it; 805 MB of weights do not fit L2, no flush needed.
    rnd = __import__("random").Random(MOE["seed"])
    counts = [rnd.randint(1, 64) for _ in range(E)]
    keep, args = moe_setup(torch, dev, counts, K, N, MOE["seed"])
    ms = _time(lambda: fb.group_bfgemm(*args, use_small_m=True), torch)
    Td = sum(counts)
    nbytes = 2 * (Td * K + E * K * N + Td * N)
    out["group_bfgemm_moe64_decode"] = {"tflops": 2.0 * Td * N * K / (ms * 1e-3) / 1e12, "ms": ms, "tokens": Td,
                                        "gbs": nbytes / (ms * 1e-3) / 1e9, "bound": "hbm",
                                        "frac": nbytes / (ms * 1e-3) / 1e9 / hbm, "peak": hbm}
    del keep, args
    # matrix-vector products (the callers' decode-time shape): A read once, HBM bound
    for op, dt in (("bfgemv", torch.bfloat16), ("sgemv", torch.float32)):
        for trans in (0, 1):
            m = n = 16384
            g = torch.Generator(device=dev).manual_seed(5)
            A = torch.randn(m, n, generator=g, device=dev).to(dt)
            x = torch.randn(n, generator=g, device=dev).to(dt)
            y = torch.zeros(m, device=dev, dtype=dt)
            fn = getattr(fb, op)
            ms = _time(lambda: fn(trans, m, n, 1.0, A, n, x, 1, 0.0, y, 1), torch)
            gbs = A.element_size() * (m * n + m + n) / (ms * 1e-3) / 1e9
            out["%s_16384_%s" % (op, "nt"[trans])] = {"ms": ms, "gbs": gbs, "bound": "hbm", "frac": gbs / hbm, "peak": hbm}
            del A, x, y
    return out


def moe_token_counts(torch):
    w = torch.arange(1, MOE["experts"] + 1, dtype=torch.float64) ** -MOE["zipf"]
    gc = torch.Generator().manual_seed(MOE["seed"])
    return torch.multinomial(w / w.sum(), MOE["tokens"], replacement=True, generator=gc).bincount(minlength=MOE["experts"]).tolist()


def run_grouped(args, rank, world, local_rank):
    """The grouped MoE workload as the benchmarked one: ``group_bfgemm`` over 64 experts.  With N > 1 ranks
    the groups are dealt out by FLOPs (largest first, oversize groups cut into row slices); every rank
    holds the tokens and weights, runs its pieces, and nothing is exchanged."""
    import torch

    import flagblas_b200 as fb
    from flagblas_b200 import dist as fbdist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as tdist

        tdist.init_process_group("nccl", device_id=dev)
    E, K, N, T = MOE["experts"], MOE["k"], MOE["n"], MOE["tokens"]
    ms_ = moe_token_counts(torch)
    g = torch.Generator(device=dev).manual_seed(MOE["seed"])
    A = torch.randn(T, K, generator=g, device=dev).bfloat16()
    B = (torch.randn(E * K, N, generator=g, device=dev) * 0.02).bfloat16()
    O = torch.full((T, N), float("nan"), device=dev, dtype=torch.bfloat16)
    starts = [sum(ms_[:e]) for e in range(E)]
    a_ptrs = [A.data_ptr() + s * K * 2 for s in starts]
    b_ptrs = [B.data_ptr() + e * K * N * 2 for e in range(E)]
    o_ptrs = [O.data_ptr() + s * N * 2 for s in starts]
    plan = fbdist.plan_group_shards(ms_, [N] * E, [K] * E, world, row_align=256)
    imbalance = fbdist.plan_imbalance(plan, ms_, [N] * E, [K] * E)
    arrays, pieces = fbdist.shard_group_arrays(plan[rank], a_ptrs, b_ptrs, o_ptrs, o_ptrs, ms_, [N] * E, [K] * E,
                                               [K] * E, [N] * E, [N] * E, 2, dev)
    rows_here = sum(r for _, _, r in plan[rank])

    def step():
        if pieces:
            fb.group_bfgemm(O, *arrays, pieces, rows_here, N, K, 1.0, 0.0)

    def barrier():
        if use_dist:
            tdist.barrier()
        torch.cuda.synchronize()

    def maxed(ms):
        if use_dist:
            t = torch.tensor([ms], device=dev)
            tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
            return float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert fb.device_status() == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    ms_step = maxed(e0.elapsed_time(e1)) / args.steps
    flops = 2.0 * T * N * K
    value = flops / (ms_step * 1e-3) / 1e12
    status = fb.device_status()

    hA, hB = A.cpu().pin_memory(), B.cpu().pin_memory()
    hO = torch.empty(O.shape, dtype=O.dtype).pin_memory()

    def e2e_step():
        A.copy_(hA, non_blocking=True)
        B.copy_(hB, non_blocking=True)
        step()
        hO.copy_(O, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    barrier()
    e0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = maxed(e0.elapsed_time(e1) / args.e2e_steps)
    if rank == 0:
        peak, peak_src = measured_peak()
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": MOE["name"], "op": "group_bfgemm", "experts": E, "k": K, "n": N, "tokens": T,
                       "token_counts": "Multinomial(32768, Zipf(1.2)) seed 3", "alpha": 1.0, "beta": 0.0,
                       "accumulate": "f32",
                       "parallelism": "single GPU" if world == 1 else "groups dealt by FLOPs over %d GPUs (row slices of oversize groups), no collective; planned imbalance %.3f" % (world, imbalance),
                       "l2": "per-GPU inputs (%.0f MiB) larger than L2; no flush between steps" % ((A.numel() + B.numel() + O.numel()) * 2 / 2**20)},
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                         "frac": value / world / peak, "traffic": ncu_traffic(MOE["name"]) if world == 1 else None,
                         "peak_source": peak_src, "frac_of_nominal_2250": value / world / 2250.0, "per_gpu": True},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (A.numel() + B.numel()) * 2, "d2h_bytes_per_step": O.numel() * 2,
                    "ms_per_step": e2e_ms},
            "gpu_launches": 2 * args.steps,  # table builder + GEMM kernel per step
            "clocks": clk.summary(), "device_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import cpu_baseline

            tf, rows, secs, threads = cpu_baseline.time_dense_rows(T, N, K, 0, 0, target_seconds=12.0, seed=MOE["seed"], scale=1.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": "torch.matmul fp32 on %d token rows against one expert's [4096, 1536] weights (inputs upcast), repeated for %.1f s" % (rows, secs)}
        emit(line)
    if use_dist:
        tdist.destroy_process_group()


GEMV = {  # name: (operator, torch dtype name, trans, m, n)
    "bfgemv_16384_n": ("bfgemv", "bfloat16", 0, 16384, 16384), "bfgemv_16384_t": ("bfgemv", "bfloat16", 1, 16384, 16384),
    "sgemv_16384_n": ("sgemv", "float32", 0, 16384, 16384), "sgemv_16384_t": ("sgemv", "float32", 1, 16384, 16384),
}


def run_gemv(args, local_rank):
    """Matrix-vector workloads (single GPU): y = A x or A^T x, A 16384 x 16384 read once -- HBM bound."""
    import torch

    import flagblas_b200 as fb

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    op, dtn, trans, m, n = GEMV[args.workload]
    dt = getattr(torch, dtn)
    g = torch.Generator(device=dev).manual_seed(5)
    A = torch.randn(m, n, generator=g, device=dev).to(dt)
    x = torch.randn(m if trans else n, generator=g, device=dev).to(dt)
    y = torch.full((n if trans else m,), float("nan"), device=dev, dtype=dt)
    fn = getattr(fb, op)

    def step():
        fn(trans, m, n, 1.0, A, n, x, 1, 0.0, y, 1)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / args.steps
    nbytes = A.element_size() * (m * n + m + n)
    hA = A.cpu().pin_memory()
    hy = torch.empty(y.shape, dtype=dt).pin_memory()

    def e2e_step():
        A.copy_(hA, non_blocking=True)
        step()
        hy.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    e0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm, src = float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except (OSError, KeyError, ValueError):
        hbm, src = 6650.0, "fallback"
    gbs = nbytes / (ms_step * 1e-3) / 1e9
    ws = fb.c_operators.gemv_workspace_bytes({"bfloat16": 3, "float32": 0}[dtn], trans, m, n)
    line = {
        "metric": "gemm_tflops", "value": 2.0 * m * n / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": {"bfloat16": "bf16", "float32": "f32"}[dtn], "data": "synthetic",
        "config": {"workload": args.workload, "op": op, "trans": trans, "m": m, "n": n, "alpha": 1.0, "beta": 0.0,
                   "l2": "A (%.0f MiB) larger than L2; no flush between steps" % (A.numel() * A.element_size() / 2**20)},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                     "traffic": ncu_traffic(args.workload), "peak_source": src},
        "e2e": {"value": 2.0 * m * n / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": A.numel() * A.element_size(), "d2h_bytes_per_step": y.numel() * y.element_size(),
                "ms_per_step": e2e_ms},
        "gpu_launches": args.steps * (2 if ws else 1), "clocks": clk.summary(), "device_status": fb.device_status(),
    }
    emit(line)


def dense_config(workload, world, gather=False):
    """The ``config`` object of a dense workload's line: the same in this arm and in the reference arm."""
    op, kind, ta, tb, m, n, k, alpha, beta, sa, sb, seed = WORKLOADS[workload]
    esz = 4 if kind in ("tf32", "fp32") else 2
    mib = (m * k + k * n + m * n) * esz / 2**20
    return {"workload": workload, "op": op, "m": m, "n": n, "k": k, "transa": ta, "transb": tb, "alpha": alpha,
            "beta": beta, "accumulate": "f32",
            "parallelism": "single GPU" if world == 1 else "N-split of C columns over %d GPUs, no collective%s" % (world, " + all-gather" if gather else ""),
            "l2": "per-GPU inputs (%.0f MiB) %s L2; no flush between steps" % (mib, "larger than" if mib * 2**20 > 126e6 else "NOT larger than")}


def moe_sharded(fb, fbdist, torch, dev, rank, world, timed):
    """The grouped MoE workload on `world` ranks: groups dealt by FLOPs (row slices of oversize groups), every rank
    holds tokens and weights, nothing is exchanged.  Whole-job TFLOP/s from the max-over-ranks time."""
    E, K, N, T = MOE["experts"], MOE["k"], MOE["n"], MOE["tokens"]
    ms_ = moe_token_counts(torch)
    (A, B, O), _ = moe_setup(torch, dev, ms_, K, N, MOE["seed"])
    starts = [sum(ms_[:e]) for e in range(E)]
    a_ptrs = [A.data_ptr() + s * K * 2 for s in starts]
    b_ptrs = [B.data_ptr() + e * K * N * 2 for e in range(E)]
    o_ptrs = [O.data_ptr() + s * N * 2 for s in starts]
    plan = fbdist.plan_group_shards(ms_, [N] * E, [K] * E, world, row_align=256)
    arrays, pieces = fbdist.shard_group_arrays(plan[rank], a_ptrs, b_ptrs, o_ptrs, o_ptrs, ms_, [N] * E, [K] * E,
                                               [K] * E, [N] * E, [N] * E, 2, dev)
    rows_here = sum(r for _, _, r in plan[rank])

    def step():
        if pieces:
            fb.group_bfgemm(O, *arrays, pieces, rows_here, N, K, 1.0, 0.0)

    for _ in range(3):
        step()
    ms = timed(step, 10)
    peak, _ = measured_peak()
    tf = 2.0 * T * N * K / (ms * 1e-3) / 1e12
    rec = {"tflops": tf, "ms": ms, "bound": "tensor", "frac": tf / world / peak, "peak": peak, "per_gpu": True,
           "planned_imbalance": fbdist.plan_imbalance(plan, ms_, [N] * E, [K] * E)}
    if pieces:
        # tables built once per routing, reused by every call (group_prepare / plan.run)
        gplan = fb.group_prepare("group_bfgemm", *arrays, pieces, rows_here, N, K)
        run = lambda: gplan.run(O, 1.0, 0.0)  # noqa: E731
    else:
        run = lambda: None  # noqa: E731
    for _ in range(3):
        run()
    ms2 = timed(run, 10)
    rec["prepared"] = {"tflops": 2.0 * T * N * K / (ms2 * 1e-3) / 1e12, "ms": ms2}
    return rec


def run_reference(args, rank, world):
    """Reference arm: the path on the host cores (torch.matmul fp32 over a bounded row sample)."""
    if rank != 0:
        return
    from oracle import cpu_baseline

    if args.workload in GEMV:
        op_, _, tr_, m_, n_ = GEMV[args.workload]
        WORKLOADS[args.workload] = (op_, "fp32", 0, 0, m_, 1, n_, 1.0, 0.0, 1.0, 1.0, 5)   # A x as an [m, n] x [n, 1] product
    if args.workload == MOE["name"]:
        WORKLOADS[MOE["name"]] = ("group_bfgemm", "bf16", 0, 0, MOE["tokens"], MOE["n"], MOE["k"], 1.0, 0.0, 1.0, 0.02, MOE["seed"])

    # the same `config` object as this repo's arm prints for the workload
    ref_config = (dense_config(args.workload, world, args.gather) if (args.workload in WORKLOADS and args.workload not in GEMV
                                                                      and args.workload != MOE["name"])
                  else {"workload": args.workload})
    op, kind, ta, tb, m, n, k, alpha, beta, sa, sb, seed = WORKLOADS[args.workload]
    per_step = max(0.5, min(20.0, 60.0 / max(1, args.steps + args.warmup)))  # the whole run stays near a minute
    vals, rows, threads = [], 0, 1
    for i in range(args.warmup + args.steps):
        tf, rows, secs, threads = cpu_baseline.time_dense_rows(m, n, k, ta, tb, target_seconds=per_step, seed=seed, scale=sa)
        if i >= args.warmup:
            vals.append((tf, secs))
    tf = sum(v[0] for v in vals) / len(vals)
    sample = "torch.matmul fp32 on %d of %d output rows of %s, repeated for ~%.0f s per step (inputs upcast)" % (rows, m, args.workload, per_step)
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * 2.0 * rows * n * k / (tf * 1e12),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": ref_config,
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS) + [MOE["name"]] + sorted(GEMV))
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", action="store_true", help="N>1: all-gather C over NCCL inside the timed step")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the brief runs of the other workloads")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second back-to-back loop")
    args = ap.parse_args()
    claim_stdout()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)
    if args.workload == MOE["name"]:
        run_grouped(args, rank, world, local_rank)
        return
    if args.workload in GEMV:
        if rank == 0:
            run_gemv(args, local_rank)
        return

    import torch

    import flagblas_b200 as fb
    from flagblas_b200 import dist as fbdist

    assert torch.cuda.is_available(), "bench.py measures the CUDA path; no GPU visible"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as tdist

        tdist.init_process_group("nccl", device_id=dev)

    op, kind, ta, tb, m, n, k, alpha, beta, sa, sb, seed = WORKLOADS[args.workload]
    dt = {"fp16": torch.float16, "bf16": torch.bfloat16, "tf32": torch.float32, "fp32": torch.float32}[kind]
    g = torch.Generator(device=dev).manual_seed(seed)  # same seed on every rank: the same global A, B, C
    A = (torch.randn((k, m) if ta else (m, k), generator=g, device=dev) * sa).to(dt)
    B = (torch.randn((n, k) if tb else (k, n), generator=g, device=dev) * sb).to(dt)
    C = (torch.randn(m, n, generator=g, device=dev) * 0.02).to(dt) if beta != 0 else torch.full((m, n), float("nan"), device=dev, dtype=dt)
    lda, ldb, ldc = A.shape[1], B.shape[1], n
    n0, n1 = fbdist.column_ranges(n, world)[rank]
    nl = n1 - n0
    opfn = getattr(fb, op)

    # Device-resident step.  N > 1: column-sharded in place -- every rank holds full-size A, B and C with their
    # original leading dimensions and computes its column block of C (the shard of B / C is a strided view; nothing
    # is copied or exchanged).  --gather adds the all-gather that completes C on every rank.
    def step():
        if world == 1:
            opfn(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
        elif args.gather:
            fbdist.sharded_gemm(op, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, rank, world)
            fbdist.all_gather_columns(C, m, n, ldc, rank, world)
        else:
            fbdist.sharded_gemm(op, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, rank, world)

    def barrier():
        if use_dist:
            tdist.barrier()
        torch.cuda.synchronize()

    def maxed(ms):
        if use_dist:
            t = torch.tensor([ms], device=dev)
            tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed(fn, steps, sampler=None):
        """ms per step of `steps` back-to-back calls, barrier + synchronize on both sides, max over ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return maxed(e0.elapsed_time(e1)) / steps

    for _ in range(args.warmup):
        step()
    barrier()
    assert fb.device_status() == 0
    with ClockSampler(local_rank) as clk:
        ms_step = timed(step, args.steps)
    flops = 2.0 * m * n * k
    value = flops / (ms_step * 1e-3) / 1e12
    status = fb.device_status()

    # ---- sustained: the same step back to back for at least two seconds (the clock sags under load), with the SM
    # clock sampled over that window
    # ---- context: cuBLAS (torch.matmul) on the same box, operands and loop length, after the timed region
    cublas_tflops = None
    if world == 1 and m * n <= 8192 * 8192:
        try:
            time.sleep(0.3)
            opA, opB = (A.t() if ta else A), (B.t() if tb else B)
            tmp = torch.empty((m, n), device=dev, dtype=dt)
            torch.backends.cuda.matmul.allow_tf32 = kind == "tf32"
            for _ in range(3):
                torch.matmul(opA, opB, out=tmp)
            cublas_tflops = flops / (timed(lambda: torch.matmul(opA, opB, out=tmp), min(args.steps, 20)) * 1e-3) / 1e12
            torch.backends.cuda.matmul.allow_tf32 = False
            del tmp
            time.sleep(0.3)
        except Exception:
            cublas_tflops = None

    sustained = None
    if not args.no_sustained:
        n_sus = max(args.steps, int(2200.0 / ms_step) + 1)
        time.sleep(0.5)
        with ClockSampler(local_rank, period=0.01) as sclk:
            sus_ms = timed(step, n_sus)
        sus_peak, sus_src = measured("bf16_tflops_sustained", 1400.0)
        if kind == "fp32":
            sus_peak, sus_src = 148 * 128 * 2 * 1.965e9 / 1e12, "nominal FFMA rate at the maximum SM clock"
        elif kind == "tf32":
            sus_peak, sus_src = sus_peak / 2, "assumed: " + sus_src + " / 2 (no measured TF32 figure)"
        sus_val = flops / (sus_ms * 1e-3) / 1e12
        sustained = {"value": sus_val, "unit": "TFLOP/s", "steps": n_sus, "seconds": sus_ms * n_sus * 1e-3,
                     "ms_per_step": sus_ms, "clocks": sclk.summary(), "peak": sus_peak, "peak_source": sus_src,
                     "frac": sus_val / world / sus_peak, "per_gpu": True}
        time.sleep(0.5)

    # ---- N > 1: what the optional all-gather of C costs, serial and overlapped by row blocks; and the same
    # column block computed from densely pitched local shards of B and C (what a tensor-parallel caller holds)
    gather = None
    if use_dist and not args.gather:
        try:
            def serial():
                fbdist.sharded_gemm(op, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, rank, world)
                fbdist.all_gather_columns(C, m, n, ldc, rank, world)

            def overlapped():
                fbdist.sharded_gemm_gather(op, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, rank, world)

            for fn in (serial, overlapped):
                fn()
            gather = {"ms_gemm_only": ms_step, "ms_gemm_then_all_gather": timed(serial, 5),
                      "ms_all_gather_overlapped_by_row_blocks": timed(overlapped, 5),
                      "bytes_per_rank": m * nl * A.element_size()}
        except Exception as exc:  # the headline line must survive a failing side measurement
            gather = {"error": repr(exc)[:200]}

    # ---- end to end: host buffers in, host buffer out, through the library's host-memory entry.  N > 1: every rank
    # owns the densely pitched column shards of B and C; of A it copies 1/N of every row block from the host and the
    # ranks complete the block with an all-gather over NVLink.
    esz = A.element_size()
    if world > 1:
        Bl = (B[n0:n1] if tb else B[:, n0:n1]).contiguous()
        Cl = C[:, n0:n1].contiguous()
    else:
        Bl, Cl = B, C
    ldbl, ldcl = Bl.shape[1], Cl.shape[1]
    from flagblas_b200 import host as fbhost

    hA, hB = A.cpu().pin_memory(), Bl.cpu().pin_memory()
    hC = torch.empty(Cl.shape, dtype=dt).pin_memory()

    def e2e_step():
        fbhost.gemm_from_host_sharded(op, ta, tb, m, nl, k, alpha, hA, lda, hB, ldbl, beta, hC, ldcl, A, Bl, Cl, rank, world)
        torch.cuda.synchronize()

    e2e_step()
    # the host result of the end-to-end call against this rank's device-resident result of the same product
    if beta == 0:
        dev_ref = Cl.clone()
        if world > 1:
            opfn(ta, tb, m, nl, k, alpha, A, lda, Bl, ldbl, beta, dev_ref, ldcl)
        else:
            step()
            dev_ref = C.clone()
        torch.cuda.synchronize()
        e2e_checked = bool(torch.allclose(hC.to(dev).float(), dev_ref.float(), rtol=2e-3, atol=2e-3 * float(k) ** 0.5))
        if use_dist:  # true only if it holds on every rank
            t = torch.tensor([1 if e2e_checked else 0], device=dev)
            tdist.all_reduce(t, op=tdist.ReduceOp.MIN)
            e2e_checked = bool(t.item())
    else:
        e2e_checked = None  # (C is updated in place: every step changes the operand)
    e2e_ms = timed(e2e_step, args.e2e_steps)
    a_rows_from_host = (A.numel() // world) if (world > 1 and ta == 0 and m % world == 0) else A.numel()
    h2d = world * a_rows_from_host * esz + (n * k + (m * n if beta != 0 else 0)) * esz   # whole job, all ranks
    d2h = m * n * esz

    # ---- the other workloads, briefly (informational)
    others = {}
    if not args.no_other_configs:
        if world == 1:
            others = other_configs(fb, torch, dev)
        else:
            try:
                others = {MOE["name"]: moe_sharded(fb, fbdist, torch, dev, rank, world, timed)}
            except Exception as exc:
                others = {MOE["name"]: {"error": repr(exc)[:200]}}

    if rank == 0:
        peak, peak_src = measured_peak()
        bound = "tensor"
        if kind == "fp32":    # IEEE fp32 runs on the CUDA cores: SMs x FP32 lanes x 2 FLOP x max SM clock
            peak, peak_src, bound = 148 * 128 * 2 * 1.965e9 / 1e12, "nominal FFMA rate at the maximum SM clock", "fp32 FFMA"
        elif kind == "tf32":  # no measured TF32 figure: half the measured bf16 rate
            peak, peak_src = peak / 2, "assumed: " + peak_src + " / 2 (no measured TF32 figure)"
        traffic = ncu_traffic(args.workload) if world == 1 else None
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": {"fp16": "f16", "bf16": "bf16", "tf32": "tf32", "fp32": "f32"}[kind],
            "data": "synthetic",
            "config": dense_config(args.workload, world, args.gather),
            "roofline": {"bound": bound, "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                         "frac": value / world / peak, "traffic": traffic, "peak_source": peak_src,
                         "cublas_same_operands_tflops": cublas_tflops,
                         "frac_of_nominal_2250": value / world / 2250.0 if kind in ("fp16", "bf16") else None, "per_gpu": True},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "checked_against_device_result": e2e_checked},
            "gpu_launches": args.steps,
            "other_configs": others,
            "clocks": clk.summary(),
            "device_status": status,
        }
        if sustained is not None:
            line["sustained"] = sustained
        if gather is not None:
            line["gather"] = gather
        if world == 1 and not args.no_cpu_baseline:
            from oracle import cpu_baseline

            tf, rows, secs, threads = cpu_baseline.time_dense_rows(m, n, k, ta, tb, target_seconds=12.0, seed=seed, scale=sa)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": "torch.matmul fp32 on %d of %d output rows of %s (inputs upcast), repeated for %.1f s" % (rows, m, args.workload, secs)}
        emit(line)
    if use_dist:
        tdist.destroy_process_group()


if __name__ == "__main__":
    main()
