"""CUDA-event timing of the tcgen05 GEMM against torch.matmul (cuBLAS) on the per-rank shapes of
the Llama-3-8B / 70B layers.  L2 is flushed (256 MB memset) between timed iterations; median of 10.

    python -m lightllm_b200.utils.gemm_bench [--quick]
"""
from __future__ import annotations

import argparse
import json

import torch


def timeit(fn, flush, n=10, reps=8):
    """Median over n samples of (time of `reps` back-to-back calls fn(i)) / reps.  fn(i) should use the
    i-th copy of its operands so that consecutive calls do not hit each other's data in L2; the launches
    are queued behind a 256 MB memset, so host launch latency is hidden."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    ts.sort()
    return ts[len(ts) // 2]


def main():
    from lightllm_b200 import ops

    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--stream-k", action="store_true", help="also time the stream-K schedule")
    ap.add_argument("--reps", type=int, default=8, help="back-to-back launches per timed sample")
    a = ap.parse_args()
    dev = torch.device("cuda")
    shapes = [(16384, 6144, 4096), (16384, 4096, 4096), (16384, 28672, 4096), (16384, 4096, 14336),
              (256, 6144, 4096), (256, 4096, 4096), (256, 28672, 4096), (256, 4096, 14336), (256, 128256, 4096),
              (64, 6144, 4096), (64, 4096, 14336), (8192, 8192, 8192), (4096, 1280, 8192), (4096, 8192, 1024),
              (256, 1280, 8192), (256, 8192, 1024), (256, 7168, 8192), (256, 8192, 3584)]
    if a.quick:
        shapes = shapes[:9]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for M, N, K in shapes:
        reps = a.reps
        copies = max(1, min(reps, int((2 << 30) // max((M * K + N * K) * 2, 1))))
        xs = [(torch.randn(M, K, device=dev) * 0.5).bfloat16() for _ in range(copies)]
        ws = [(torch.randn(N, K, device=dev) * 0.1).bfloat16() for _ in range(copies)]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        row = {"M": M, "N": N, "K": K}
        t = timeit(lambda i: torch.matmul(xs[i % copies], ws[i % copies].t(), out=out), flush, reps=reps)
        row["cublas_ms"] = round(t, 4)
        row["cublas_tflops"] = round(2 * M * N * K / t / 1e9, 1)
        variants = {"auto": dict(), "dp256": dict(bn=256, stream_k=0), "dp128": dict(bn=128, stream_k=0),
                    "dp64": dict(bn=64, stream_k=0), "pair": dict(bn=512, stream_k=0)}
        if a.stream_k:
            variants.update({"sk256": dict(bn=256, stream_k=1), "sk128": dict(bn=128, stream_k=1)})
        done = []
        for name, kw in variants.items():
            if kw.get("stream_k") == 1 and ((M + 127) // 128) * ((N + kw["bn"] - 1) // kw["bn"]) > 8192:
                continue  # more tiles than arrival counters
            if kw.get("bn") == 512 and (M < 256 or N < 256):
                continue
            t = timeit(lambda i: ops.gemm(xs[i % copies], ws[i % copies], out=out, **kw), flush, reps=reps)
            row[f"{name}_ms"] = round(t, 4)
            done.append(name)
        best = min(row[f"{n}_ms"] for n in done)
        row["auto_tflops"] = round(2 * M * N * K / row["auto_ms"] / 1e9, 1)
        row["best_tflops"] = round(2 * M * N * K / best / 1e9, 1)
        row["auto_weight_gbs"] = round(N * K * 2 / row["auto_ms"] / 1e6, 1)
        row["auto_vs_cublas"] = round(row["cublas_ms"] / row["auto_ms"], 3)
        print(json.dumps(row), flush=True)
    print("gemm wait status", int(ops.gemm_status(dev).item()))


if __name__ == "__main__":
    main()
