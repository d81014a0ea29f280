"""CUDA-event timing of the attention kernels on Llama-3-8B head geometry.

    python -m lightllm_b200.benchmark.attn_bench [--B 16 --len 1024 --reps 5]            # causal prefill (tcgen05 kernel;
                                                                                      # LLB_ATTN_TC=0: mma.sync kernel)
    python -m lightllm_b200.benchmark.attn_bench --decode --B 256 --len 1024 [--int8kv]  # split-KV decode, bf16 or int8 pool
"""
from __future__ import annotations

import argparse
import json

import torch


def bench_decode(a, dev, Hq, Hkv, D, B, L):
    from lightllm_b200 import ops
    from lightllm_b200.common.mem_manager import Int8KVMemoryManager
    from lightllm_b200.ops import kv_quant

    slots = B * L
    vals = (torch.randn(slots + 1, 2 * Hkv, D, device=dev) * 0.5).bfloat16()
    if a.int8kv:
        mm = Int8KVMemoryManager(slots, torch.bfloat16, Hkv, D, 1, dev)
        kv = mm.layer(0)
        kv_quant.quant_store_(kv, vals, torch.arange(slots + 1, dtype=torch.int32, device=dev))
        row_bytes = 2 * Hkv * (D + kv_quant.PAD)
    elif a.fp8kv:
        from lightllm_b200.common.mem_manager import Fp8KVMemoryManager

        mm = Fp8KVMemoryManager(slots, torch.bfloat16, Hkv, D, 1, dev)
        mm.scales.fill_(0.01)
        kv = mm.layer(0)
        kv_quant.quant_store_(kv, vals, torch.arange(slots + 1, dtype=torch.int32, device=dev))
        row_bytes = 2 * Hkv * D
    else:
        kv, row_bytes = vals, 2 * Hkv * D * 2
    r2t = torch.arange(slots, dtype=torch.int32, device=dev).view(B, L)
    b_req = torch.arange(B, dtype=torch.int32, device=dev)
    seq = torch.full((B,), L, dtype=torch.int32, device=dev)
    q = torch.randn(B, Hq * D, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        ops.gqa_decode(q, kv, r2t, b_req, seq, Hq, Hkv, D, L)
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.gqa_decode(q, kv, r2t, b_req, seq, Hq, Hkv, D, L)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = ts[len(ts) // 2]
    print(json.dumps({"decode": True, "int8kv": bool(a.int8kv), "fp8kv": bool(a.fp8kv), "B": B, "ctx": L, "ms": round(t, 4),
                      "kv_gb": round(slots * row_bytes / 1e9, 3), "gbs": round(slots * row_bytes / t / 1e6, 1)}))


def main():
    from lightllm_b200 import ops

    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--len", type=int, default=1024)
    ap.add_argument("--ready", type=int, default=0, help="cached prefix length of every request")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--decode", action="store_true", help="time decode attention (one query token per request)")
    ap.add_argument("--int8kv", action="store_true", help="decode over the int8 pool")
    ap.add_argument("--fp8kv", action="store_true", help="decode over the fp8 (e4m3, static per-head scales) pool")
    a = ap.parse_args()
    dev = torch.device("cuda")
    Hq, Hkv, D, B, L, R = a.hq, a.hkv, 128, a.B, a.len, a.ready
    if a.decode:
        return bench_decode(a, dev, Hq, Hkv, D, B, L)
    T = B * L
    total = B * (L + R)
    kv = (torch.randn(total + 1, 2 * Hkv, D, device=dev) * 0.5).bfloat16()
    r2t = torch.arange(total, dtype=torch.int32, device=dev).view(B, L + R)
    b_req = torch.arange(B, dtype=torch.int32, device=dev)
    cu = torch.arange(0, T + 1, L, dtype=torch.int32, device=dev)
    ready = torch.full((B,), R, dtype=torch.int32, device=dev)
    q = torch.randn(T, Hq * D, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        ops.gqa_prefill(q, kv, r2t, b_req, cu, ready, Hq, Hkv, D, L)
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.gqa_prefill(q, kv, r2t, b_req, cu, ready, Hq, Hkv, D, L)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = ts[len(ts) // 2]
    flops = 4 * B * Hq * D * (L * L / 2 + L * R)
    print(json.dumps({"B": B, "len": L, "ready": R, "ms": round(t, 4), "tflops": round(flops / t / 1e9, 1)}))


if __name__ == "__main__":
    main()
