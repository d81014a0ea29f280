"""Times the fused NVLink all-reduce + residual + RMSNorm kernel against NCCL all-reduce followed by the
standalone add+RMSNorm kernel, over message sizes, grid sizes and both algorithms.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29621 -m lightllm_b200.benchmark.comm_bench

CUDA events on the launching stream, 3 warm-up and 30 timed calls back to back, max over ranks.  Both sides
include their host launch cost (two launches for the NCCL side, one for the fused kernel).  The first block
(`graph ...` lines; LLB_COMM_BENCH=graph prints only it) times the decode-sized calls inside CUDA graphs instead.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def graph_latency(ps, say):
    """Per-call device time of the decode-sized reductions inside a CUDA graph (20 calls per replay, as the decode
    step issues them: no host launch cost), next to the whole row-parallel step GEMM -> reduce + residual + norm for
    the Llama-3-8B o_proj / down_proj shards of this world size.  Max over ranks."""
    from .. import ops
    from ..parallel.fused import FusedTP

    dev, world = ps.device, ps.world_size
    H, CALLS = 4096, 20

    def timeit_graph(fn, n=10):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(4):      # an even number of calls keeps the two buffer parities aligned
                fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(CALLS):
                fn()
        ts = []
        for _ in range(n):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / CALLS * 1e3)
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del g
        return float(t)

    f = FusedTP(ps, max_tokens=1024, hidden=H)
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    for T in (16, 64, 256, 1024):
        res = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        y = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        row = {"T": T, "MB_per_rank": round(T * H * 2 / 1e6, 2)}
        row["nccl_ar_norm"] = timeit_graph(lambda: (dist.all_reduce(y), ops.add_rmsnorm_(res, y, w, 1e-5)))
        for name, one in (("fused_one_shot", 1), ("fused_two_shot", 0)):
            f.force_one_shot = one
            row[name] = timeit_graph(lambda: f.reduce_residual_norm(f.partial_out(T, H), res, w, 1e-5))
        f.force_one_shot = None
        row["tpsp_rs_norm_ag"] = timeit_graph(lambda: f.tpsp_reduce(f.partial_out(T, H), res, w, 1e-5))
        # the whole row-parallel step on the o_proj and down_proj shards
        for tag, K in (("o", 4096 // world), ("down", 14336 // world)):
            a = (torch.randn(T, K, device=dev) * 0.1).bfloat16()
            wt = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
            row[f"{tag}_gemm_alone"] = timeit_graph(lambda: ops.gemm(a, wt))
            f.force_one_shot = 0
            row[f"{tag}_gemm+two_shot"] = timeit_graph(
                lambda: f.reduce_residual_norm(ops.gemm(a, wt, out=f.partial_out(T, H)), res, w, 1e-5))
            f.force_one_shot = 1
            if f.can_push(T, H):
                row[f"{tag}_gemm_push+reduce"] = timeit_graph(
                    lambda: f.reduce_pushed(*f.gemm_push(a, wt), res, w, 1e-5))
            f.force_one_shot = None
            row[f"{tag}_gemm+tpsp"] = timeit_graph(
                lambda: f.tpsp_reduce(ops.gemm(a, wt, out=f.partial_out(T, H)), res, w, 1e-5))
            row[f"{tag}_gemm+nccl_ar_norm"] = timeit_graph(
                lambda: ops.add_rmsnorm_(res, (lambda o: (dist.all_reduce(o), o)[1])(ops.gemm(a, wt)), w, 1e-5))
        say("graph " + " ".join(f"{k}={v:.1f}" if isinstance(v, float) else f"{k}={v}" for k, v in row.items())
            + f" status={f.status()}")
    f.close()


def main():
    from .. import ops
    from ..parallel import dist as pdist
    from ..parallel.fused import FusedTP

    ps = pdist.init_from_env()
    rank = ps.global_rank

    def timeit(fn, n=30):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device=ps.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def say(msg):
        if rank == 0:
            print(msg, flush=True)

    say(f"world={ps.world_size} NCCL_NVLS_ENABLE={os.environ.get('NCCL_NVLS_ENABLE', 'unset')}")
    if os.environ.get("LLB_COMM_BENCH", "all") in ("all", "graph"):
        graph_latency(ps, say)
    if os.environ.get("LLB_COMM_BENCH", "all") == "graph":
        pdist.destroy(hard_exit_on_hang=True)
        return
    for H, Ts in ((1024, (256, 4096)), (4096, (256, 2048, 16384)), (8192, (256, 8192))):
        f = FusedTP(ps, max_tokens=16384, hidden=H)
        w = torch.ones(H, dtype=torch.bfloat16, device=ps.device)
        for T in Ts:
            res = torch.zeros(T, H, dtype=torch.bfloat16, device=ps.device)
            y = torch.zeros(T, H, dtype=torch.bfloat16, device=ps.device)
            t_nccl = timeit(lambda: (dist.all_reduce(y), ops.add_rmsnorm_(res, y, w, 1e-5)))
            say(f"H={H} T={T} ({T * H * 2 / 1e6:.1f} MB per rank): NCCL all-reduce + add_rmsnorm {t_nccl:.1f} us")
            for one in (1, 0):
                for ctas in (148, 296, 592):
                    f.force_one_shot, f.ctas = one, ctas
                    t = timeit(lambda: f.reduce_residual_norm(f.partial_out(T, H), res, w, 1e-5))
                    say(f"   fused {'one-shot' if one else 'two-shot'} ctas={ctas}: {t:.1f} us "
                        f"({t_nccl / t:.2f}x)  status={f.status()}")
        f.close()
    pdist.destroy(hard_exit_on_hang=True)


if __name__ == "__main__":
    main()
