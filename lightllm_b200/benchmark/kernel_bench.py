"""CUDA-event timings of the non-GEMM hot kernels on serving shapes, with their roofline fractions.

    python -m lightllm_b200.benchmark.kernel_bench [--peaks MEASURED_PEAKS.json]

Each kernel: 3 warm-up launches, then the median of 10 samples of 4 back-to-back launches (operands larger than
L2 or rotated, 256 MB L2 flush before every sample).  Bytes / FLOPs are the algorithmic ones of the op.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def timeit(fn, flush, n=10, reps=4):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    ts.sort()
    return ts[len(ts) // 2] * 1e-3  # seconds


def main():
    from lightllm_b200 import ops
    from lightllm_b200.ops import mla as mla_ops
    from lightllm_b200.ops import moe as moe_ops

    ap = argparse.ArgumentParser()
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    a = ap.parse_args()
    hbm, tf = 6.65e12, 1.59e15
    if os.path.exists(a.peaks):
        p = json.load(open(a.peaks))
        hbm, tf = p.get("hbm_gbs", 6650) * 1e9, p.get("bf16_tflops", 1590) * 1e12
    dev = torch.device("cuda")
    BF = torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def report(name, t, bytes_=0, flops=0):
        r = {"kernel": name, "us": round(t * 1e6, 1)}
        if bytes_:
            r["GB/s"] = round(bytes_ / t / 1e9, 1)
            r["of_measured_hbm"] = round(bytes_ / t / hbm, 3)
        if flops:
            r["TFLOP/s"] = round(flops / t / 1e12, 1)
            r["of_measured_bf16"] = round(flops / t / tf, 3)
        rows.append(r)
        print(json.dumps(r), flush=True)

    # ---- paged GQA decode / prefill (Llama-3-8B: 32 q heads, 8 kv heads, head 128) ----
    Hq, Hkv, D = 32, 8, 128
    for B, ctx in ((256, 1024), (64, 4096)):
        slots = B * ctx
        kv = (torch.randn(slots + 1, 2 * Hkv, D, device=dev) * 0.5).to(BF)
        r2t = torch.arange(slots, dtype=torch.int32, device=dev).view(B, ctx)
        b_req = torch.arange(B, dtype=torch.int32, device=dev)
        seq = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(B, Hq * D, device=dev).to(BF)
        t = timeit(lambda: ops.gqa_decode(q, kv, r2t, b_req, seq, Hq, Hkv, D, ctx), flush)
        report(f"gqa_decode B={B} ctx={ctx}", t, bytes_=slots * 2 * Hkv * D * 2)
    for B, L in ((16, 1024), (4, 4096)):
        T = B * L
        kv = (torch.randn(T + 1, 2 * Hkv, D, device=dev) * 0.5).to(BF)
        r2t = torch.arange(T, dtype=torch.int32, device=dev).view(B, L)
        b_req = torch.arange(B, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, L, dtype=torch.int32, device=dev)
        ready = torch.zeros(B, dtype=torch.int32, device=dev)
        q = torch.randn(T, Hq * D, device=dev).to(BF)
        t = timeit(lambda: ops.gqa_prefill(q, kv, r2t, b_req, cu, ready, Hq, Hkv, D, L), flush)
        report(f"gqa_prefill B={B} len={L} (causal)", t, flops=4 * B * Hq * D * L * L / 2)

    # ---- absorbed MLA decode (DeepSeek-V3 per-rank at tp8: 16 heads, latent 512 + 64) ----
    h, kvl, rope = 16, 512, 64
    for B, ctx in ((128, 2048),):
        slots = B * ctx
        pool = (torch.randn(slots + 1, 1, kvl + rope, device=dev) * 0.3).to(BF)
        r2t = torch.arange(slots, dtype=torch.int32, device=dev).view(B, ctx)
        b_req = torch.arange(B, dtype=torch.int32, device=dev)
        seq = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
        rdy = seq - 1
        q_lat = torch.randn(B, h, kvl, device=dev).to(BF)
        q_pe = torch.randn(B, h, rope, device=dev).to(BF)
        t = timeit(lambda: mla_ops.mla_attention(q_lat, q_pe, pool, r2t, b_req, seq, cu, rdy, kvl, 0.1, False), flush)
        report(f"mla_decode B={B} ctx={ctx} heads={h}", t, bytes_=slots * (kvl + rope) * 2,
               flops=2 * B * h * ctx * (kvl + rope + kvl))

    # ---- MoE expert FFN (Qwen3-30B-A3B: 128 experts, top 8, hidden 2048, inter 768) ----
    E, k, H, I = 128, 8, 2048, 768
    w13 = (torch.randn(E, 2 * I, H, device=dev) * 0.02).to(BF)
    w2 = (torch.randn(E, H, I, device=dev) * 0.02).to(BF)
    for T in (256, 8192):
        x = torch.randn(T, H, device=dev).to(BF)
        logits = torch.randn(T, E, device=dev)
        ids, w = moe_ops.topk_softmax(logits, k, True, 1.0)
        t = timeit(lambda: moe_ops.fused_experts(x, w13, w2, ids, w, "silu"), flush)
        report(f"moe_fused_experts T={T} E={E} top{k} H={H} I={I}", t, bytes_=E * 3 * I * H * 2,
               flops=2 * T * k * 3 * I * H)
        t = timeit(lambda: moe_ops.topk_softmax(logits, k, True, 1.0), flush)
        report(f"topk_softmax T={T} E={E}", t, bytes_=T * E * 4)

    # ---- sampler and small ops at decode batch 256 ----
    V = 128256
    logits = torch.randn(256, V, device=dev)
    t = timeit(lambda: ops.sample(logits), flush)
    report("sample greedy B=256 V=128256 (fp32 logits)", t, bytes_=256 * V * 4)
    x = torch.randn(16384, 4096, device=dev).to(BF)
    wn = torch.ones(4096, device=dev).to(BF)
    t = timeit(lambda: ops.rmsnorm(x, wn, 1e-5), flush)
    report("rmsnorm T=16384 H=4096", t, bytes_=2 * x.numel() * 2)
    print(json.dumps({"peaks": {"hbm_GBs": hbm / 1e9, "bf16_TFLOPs": tf / 1e12}}))


if __name__ == "__main__":
    main()
