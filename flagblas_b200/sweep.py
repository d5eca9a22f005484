"""Shape sweep of the dense bf16 operator against ``torch.matmul`` (cuBLAS) on the current GPU.

    python -m flagblas_b200.sweep [--layout nt|nn|both] [--csv out.csv]

Times ``bfgemm`` and ``torch.matmul`` on the same operands for square problems and for the shapes of linear layers
(``m`` tokens against ``[n, k]`` weights) and prints, per shape, both times, their ratio and the achieved TFLOP/s,
then the shapes with the worst ratios and the geometric mean.  Each side is timed twice, alternating, with CUDA events
around a loop of back-to-back calls (no CUDA graph: host launch cost is part of what a caller sees), and the faster
of the two runs counts.  Small shapes follow large ones in the list, so their absolute times carry the clock the
large ones left behind; the ratios are what the sweep is for.
"""
import argparse
import statistics

import torch

import flagblas_b200 as fb

SQUARE = (256, 512, 1024, 1536, 2048, 3072, 4096, 6144, 8192, 12288, 16384)
TOKENS = (1, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384)
WEIGHTS = ((4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192), (28672, 8192), (8192, 28672), (1536, 4096),
           (6144, 4096))
ODD = ((4095, 4095, 4095), (8191, 8191, 8191), (4097, 8191, 4095), (32768, 1024, 1024), (1024, 32768, 1024),
       (1024, 1024, 32768), (100, 100, 100000), (5000, 3000, 7000), (333, 777, 1555))


def shapes():
    out = [(s, s, s) for s in SQUARE]
    out += [(m, n, k) for m in TOKENS for (n, k) in WEIGHTS]
    out += list(ODD)
    return out


def timed_us(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layout", default="both", choices=["nt", "nn", "both"])
    ap.add_argument("--csv", default=None)
    args = ap.parse_args()
    dev = "cuda"
    rows = []
    for tb in {"nt": (1,), "nn": (0,), "both": (1, 0)}[args.layout]:
        for (m, n, k) in shapes():
            if m * n * 4 + m * k * 2 + n * k * 2 > 6e9:
                continue
            a = (torch.randn(m, k, device=dev) * 0.05).bfloat16()
            b = (torch.randn((n, k) if tb else (k, n), device=dev) * 0.05).bfloat16()
            c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            bt = b.t() if tb else b
            flops = 2 * m * n * k
            iters = max(5, min(200, int(2e-2 / (flops / 1.2e15 + 8e-6))))

            def ours():
                fb.bfgemm(0, tb, m, n, k, 1.0, a, k, b, b.shape[1], 0.0, c, n)

            def ref():
                torch.matmul(a, bt, out=c)

            t_ref = timed_us(ref, iters)
            t_ours = timed_us(ours, iters)
            t_ref = min(t_ref, timed_us(ref, iters))
            t_ours = min(t_ours, timed_us(ours, iters))
            rows.append((t_ours / t_ref, m, n, k, tb, t_ours, t_ref))
            print("%6d %6d %6d %s  bfgemm %9.1f us  matmul %9.1f us  ratio %.2f  %.0f TFLOP/s" %
                  (m, n, k, "NT" if tb else "NN", t_ours, t_ref, t_ours / t_ref, flops / t_ours / 1e6), flush=True)
            del a, b, c
    assert fb.device_status() == 0
    print("== worst 20")
    for r in sorted(rows, reverse=True)[:20]:
        print("ratio %.2f  %s %s  bfgemm %.1f us  matmul %.1f us" % (r[0], r[1:4], "NT" if r[4] else "NN", r[5], r[6]))
    big = [r[0] for r in rows if 2.0 * r[1] * r[2] * r[3] >= 1e11]
    print("geometric mean of bfgemm / matmul time: %.3f over %d shapes; %.3f over the %d with at least 100 GFLOP" %
          (statistics.geometric_mean([r[0] for r in rows]), len(rows), statistics.geometric_mean(big), len(big)))
    if args.csv:
        with open(args.csv, "w") as f:
            f.write("m,n,k,layout,bfgemm_us,matmul_us,ratio\n")
            for r in rows:
                f.write("%d,%d,%d,%s,%.2f,%.2f,%.3f\n" % (r[1], r[2], r[3], "NT" if r[4] else "NN", r[5], r[6], r[0]))


if __name__ == "__main__":
    main()
