"""CUDA-event timings of the Gated DeltaNet decode step (csrc/linear_attn.cu) on Qwen3-Next shapes (16 key heads,
32 value heads, head sizes 128 / 128, convolution kernel 4) next to the torch restatement of the same step.

    python -m lightllm_b200.benchmark.linear_attn_bench [--batch 64 256] [--tp 1] [--state bf16|fp32] [--once]

3 warm-up launches, then the median of 10 samples of 4 back-to-back steps with a 256 MB L2 flush before every
sample.  Algorithmic bytes of a step: the matrix state read once and written once (B x value heads x 128 x 128
numbers) plus the convolution state; `--once` runs one step of the kernels only (the small case for a profiler).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main():
    from lightllm_b200.ops import linear_attn as la

    from .kernel_bench import timeit

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, nargs="+", default=[64, 256])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--state", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    hbm = 6.65e12
    if os.path.exists(a.peaks):
        hbm = json.load(open(a.peaks)).get("hbm_gbs", 6650) * 1e9
    dev = torch.device("cuda")
    nk, nv, dk, dv, K = 16 // a.tp, 32 // a.tp, 128, 128, 4
    C = 2 * nk * dk + nv * dv
    sdt = torch.float32 if a.state == "fp32" else torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for B in a.batch:
        g = torch.Generator(device="cpu").manual_seed(B)
        mixed = torch.randn(B, C, generator=g).to(dev)
        conv_state = torch.randn(B, C, K - 1, generator=g).to(dev, torch.bfloat16)
        conv_w = (torch.randn(C, K, generator=g) * 0.5).to(dev)
        ssm = (torch.randn(B, nv, dk, dv, generator=g) * 0.1).to(dev, sdt)
        req = torch.randperm(B, generator=g).to(dev, torch.int32)
        gate = (-torch.rand(B, nv, generator=g)).to(dev)
        beta = torch.rand(B, nv, generator=g).to(dev)

        def kernels():
            return la.conv_and_delta_step(mixed, conv_state, conv_w, ssm, req, gate, beta, nk, nv, dk, dv)

        if a.once:
            kernels()
            torch.cuda.synchronize()
            print(json.dumps({"batch": B, "ran": "one step of the two kernels"}))
            continue

        def torch_step():
            rl = req.long()
            y, new_conv = la.causal_conv_step(mixed, conv_state[rl], conv_w)
            conv_state.index_copy_(0, rl, new_conv.to(conv_state.dtype))
            kd = nk * dk
            qq = y[:, :kd].view(B, nk, dk).repeat_interleave(nv // nk, dim=1)
            kk = y[:, kd:2 * kd].view(B, nk, dk).repeat_interleave(nv // nk, dim=1)
            o, new_s = la.gated_delta_step(qq, kk, y[:, 2 * kd:].view(B, nv, dv), gate, beta, ssm[rl])
            ssm.index_copy_(0, rl, new_s.to(ssm.dtype))
            return o

        t_k = timeit(kernels, flush)
        t_t = timeit(torch_step, flush)
        nbytes = 2 * ssm.numel() * ssm.element_size() + 2 * conv_state.numel() * 2 + 2 * mixed.numel() * 4
        print(json.dumps({"batch": B, "tp": a.tp, "state": a.state, "kernels_us": round(t_k * 1e6, 1),
                          "torch_us": round(t_t * 1e6, 1), "speedup": round(t_t / t_k, 2),
                          "GB/s": round(nbytes / t_k / 1e9, 1), "of_measured_hbm": round(nbytes / t_k / hbm, 3),
                          "state_MB": round(ssm.numel() * ssm.element_size() / 1e6, 1)}))


if __name__ == "__main__":
    main()
