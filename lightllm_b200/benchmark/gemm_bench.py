"""CUDA-event timing of the tcgen05 GEMM against torch.matmul (cuBLAS) on the per-rank shapes of
the Llama-3-8B / 70B layers.  L2 is flushed (256 MB memset) between timed iterations; median of 10.

    python -m lightllm_b200.benchmark.gemm_bench [--quick]
"""
from __future__ import annotations

import argparse
import json

import torch


def timeit_graph(fn, flush, n=10, reps=8):
    """Like `timeit`, but the `reps` calls are captured in one CUDA graph and replayed, so that no host launch
    cost is in the number (what a kernel costs inside the decode graph)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(reps):
            fn(i)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    ts = []
    for _ in range(n):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    ts.sort()
    return ts[len(ts) // 2]


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


def fp8_main(a, dev):
    """fp8 block-scaled GEMM (activations already quantised) and the activation quantiser, against cuBLAS bf16 and
    the bf16 tcgen05 kernel on the same shapes (DeepSeek-V3 dense projections and one expert's matrices)."""
    from lightllm_b200 import ops
    from lightllm_b200.ops import fp8

    timer = timeit_graph if a.graph else timeit
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    shapes = [(4096, 7168, 16384), (4096, 24576, 1536), (4096, 4096, 7168), (4096, 7168, 2048), (256, 7168, 16384),
              (256, 24576, 1536), (256, 4096, 7168), (256, 7168, 2048), (8192, 8192, 8192)]
    for M, N, K in shapes:
        copies = max(1, min(a.reps, int((2 << 30) // max((M * K + N * K) * 2, 1))))
        xs = [(torch.randn(M, K, device=dev) * 0.5).bfloat16() for _ in range(copies)]
        ws = [(torch.randn(N, K, device=dev) * 0.05).bfloat16() for _ in range(copies)]
        fws = [fp8.Fp8Weight.from_float(w) for w in ws]
        qs = [fp8.quant_act(x) for x in xs]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t_cublas = timer(lambda i: torch.matmul(xs[i % copies], ws[i % copies].t(), out=out), flush, reps=a.reps)
        t_bf16 = timer(lambda i: ops.gemm(xs[i % copies], ws[i % copies], out=out), flush, reps=a.reps)
        t_fp8 = timer(lambda i: fp8.gemm_fp8_quantized(qs[i % copies][0], qs[i % copies][1], fws[i % copies], out=out),
                      flush, reps=a.reps)
        t_q = timer(lambda i: fp8.quant_act(xs[i % copies]), flush, reps=a.reps)
        fl = 2 * M * N * K / 1e9
        print(json.dumps({"M": M, "N": N, "K": K, "cublas_bf16_ms": round(t_cublas, 4), "bf16_ms": round(t_bf16, 4),
                          "fp8_ms": round(t_fp8, 4), "quant_ms": round(t_q, 4), "fp8_tflops": round(fl / t_fp8, 1),
                          "cublas_bf16_tflops": round(fl / t_cublas, 1),
                          "fp8_weight_gbs": round(N * K / t_fp8 / 1e6, 1)}), flush=True)
    print("gemm wait status", int(ops.gemm_status(dev).item()))


def main():
    from lightllm_b200 import ops

    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--stream-k", action="store_true", help="also time the stream-K schedule")
    ap.add_argument("--reps", type=int, default=8, help="back-to-back launches per timed sample")
    ap.add_argument("--decode", action="store_true", help="only the M <= 256 shapes, with the skinny-kernel variants")
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays (no host launch cost)")
    ap.add_argument("--only", default=None, help="M,N,K: run just this shape (3 plain launches of --bn, for profilers)")
    ap.add_argument("--bn", type=int, default=0, help="kernel selector passed to ops.gemm with --only")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 GEMM on DeepSeek-V3 shapes vs the bf16 kernels")
    ap.add_argument("--tp", type=int, default=0, help="with --decode: the per-rank Llama-3-8B layer shapes of a "
                                                      "tensor-parallel split over this many ranks (M = 256)")
    a = ap.parse_args()
    dev = torch.device("cuda")
    if a.fp8:
        return fp8_main(a, dev)
    if a.only:
        M, N, K = (int(v) for v in a.only.split(","))
        x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        ws = [(torch.randn(N, K, device=dev) * 0.1).bfloat16() for _ in range(3)]
        for w in ws:
            ops.gemm(x, w, bn=a.bn)
        torch.cuda.synchronize()
        print("gemm wait status", int(ops.gemm_status(dev).item()))
        return
    timer = timeit_graph if a.graph else timeit
    shapes = [(16384, 6144, 4096), (16384, 4096, 4096), (16384, 28672, 4096), (16384, 4096, 14336),
              (256, 6144, 4096), (256, 4096, 4096), (256, 28672, 4096), (256, 4096, 14336), (256, 128256, 4096),
              (64, 6144, 4096), (64, 4096, 14336), (8192, 8192, 8192), (4096, 1280, 8192), (4096, 8192, 1024),
              (256, 1280, 8192), (256, 8192, 1024), (256, 7168, 8192), (256, 8192, 3584)]
    if a.quick:
        shapes = shapes[:9]
    if a.decode:
        shapes = [sh for sh in shapes if sh[0] <= 256] + [(32, 6144, 4096), (32, 28672, 4096), (8, 4096, 14336)]
    if a.decode and a.tp > 1:
        t = a.tp
        shapes = [(256, 6144 // t, 4096), (256, 4096, 4096 // t), (256, 28672 // t, 4096), (256, 4096, 14336 // t),
                  (256, 128256 // t, 4096)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for M, N, K in shapes:
        reps = a.reps
        copies = max(1, min(reps, int((2 << 30) // max((M * K + N * K) * 2, 1))))
        xs = [(torch.randn(M, K, device=dev) * 0.5).bfloat16() for _ in range(copies)]
        ws = [(torch.randn(N, K, device=dev) * 0.1).bfloat16() for _ in range(copies)]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        row = {"M": M, "N": N, "K": K}
        t = timer(lambda i: torch.matmul(xs[i % copies], ws[i % copies].t(), out=out), flush, reps=reps)
        row["cublas_ms"] = round(t, 4)
        row["cublas_tflops"] = round(2 * M * N * K / t / 1e9, 1)
        variants = {"auto": dict(), "dp256": dict(bn=256, stream_k=0), "dp128": dict(bn=128, stream_k=0),
                    "dp64": dict(bn=64, stream_k=0), "pair": dict(bn=512, stream_k=0)}
        if M > 256:  # the same cluster kernel, one 256 x 512 (or 256 x 256) tile per CTA pair
            variants.update({"sk_n2s1": dict(bn=1021), "sk_n1s1": dict(bn=1011)})
        if M <= 256:  # skinny kernel: 1000 + 10 * accumulators + K splits
            variants.update({"sk_n1s1": dict(bn=1011), "sk_n1s2": dict(bn=1012), "sk_n1s4": dict(bn=1014),
                             "sk_n2s1": dict(bn=1021), "sk_w128s1": dict(bn=1111), "sk_w128s2": dict(bn=1112)})
        if M <= 256 and N <= 148 * 128:  # split-K without clusters: 2000 + splits (2000 = as many as fit)
            variants.update({"spk_max": dict(bn=2000), "spk_s1": dict(bn=2001), "spk_s2": dict(bn=2002),
                             "spk_s4": dict(bn=2004), "spk_s8": dict(bn=2008)})
        if ((M + 255) // 256) * ((N + 255) // 256) * 2 <= 148:  # pair tiles split through the L2 workspace
            variants.update({"psk_max": dict(bn=3000), "psk_s1": dict(bn=3001), "psk_s2": dict(bn=3002),
                             "psk_s4": dict(bn=3004), "psk_s8": dict(bn=3008)})
        if a.stream_k:
            variants.update({"sk256": dict(bn=256, stream_k=1), "sk128": dict(bn=128, stream_k=1)})
        tiled = None
        if M <= 256 and N % 128 == 0 and K % 64 == 0:  # the same kernels over the tiled weight layout
            tiled = [ops.TiledWeight(w) for w in ws]
            variants.update({"skt_n1s1": dict(bn=1011, tiled=1), "skt_n1s2": dict(bn=1012, tiled=1),
                             "skt_n1s4": dict(bn=1014, tiled=1), "skt_n2s1": dict(bn=1021, tiled=1)})
        swz = None
        if N % 256 == 0 and K % 64 == 0:  # one-CTA kernels with W as pre-swizzled tiles fetched by untiled bulk copies
            swz = [ops.TiledWeight(w, swizzle=True) for w in ws]
            variants.update({"swz256": dict(bn=256, tiled=2), "swz128": dict(bn=128, tiled=2)})
        done = []
        for name, kw in variants.items():
            kw = dict(kw)
            sel = kw.pop("tiled", 0)
            wsel = swz if sel == 2 else (tiled if sel else ws)
            if kw.get("stream_k") == 1 and ((M + 127) // 128) * ((N + kw["bn"] - 1) // kw["bn"]) > 8192:
                continue  # more tiles than arrival counters
            if kw.get("bn") == 512 and (M < 256 or N < 256):
                continue
            if 1000 <= kw.get("bn", 0) < 2000 and ((K + 63) // 64) < 4 * (kw["bn"] % 10):
                continue
            if 3000 < kw.get("bn", 0) < 3100:
                sp, pr, kbs = kw["bn"] - 3000, ((M + 255) // 256) * ((N + 255) // 256), (K + 63) // 64
                if pr * 2 * sp > 148 or -(-kbs // sp) * (sp - 1) >= kbs:
                    continue
            if 2000 < kw.get("bn", 0) < 2100:
                sp, tl, kbs = kw["bn"] - 2000, (N + 127) // 128, (K + 63) // 64
                if tl * sp > 148 or sp > (8 if M > 128 else 4) or -(-kbs // sp) * (sp - 1) >= kbs:
                    continue
            t = timer(lambda i: ops.gemm(xs[i % copies], wsel[i % copies], out=out, **kw), flush, reps=reps)
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
