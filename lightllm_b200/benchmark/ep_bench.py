"""Times the expert-parallel token exchange (dispatch -> local experts -> combine) of one MoE layer inside a CUDA
graph, for decode- and prompt-sized token counts, against the same experts run locally without an exchange.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29625 -m lightllm_b200.benchmark.ep_bench [--hidden 2048 --inter 768 --experts 128 --topk 8]

Per token count T (tokens per rank): `exchange_only` = dispatch + combine with an expert function that only copies
its rows (what the exchange itself costs), `ep_layer` = with the grouped expert GEMMs, `local_experts` = the same
number of routed rows through this rank's experts without any exchange.  Microseconds per call, 10 calls per graph
replay, median of 10 replays, max over ranks.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist


def main():
    from ..ops import moe as moe_ops
    from ..parallel import dist as pdist
    from ..parallel.ep import EPGroup

    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--tokens", default="16,64,128,256,4096")
    a = ap.parse_args()
    ps = pdist.init_from_env(dp=int(__import__("os").environ.get("WORLD_SIZE", "1")))
    dev, W, rank = ps.device, ps.world_size, ps.global_rank
    H, I, E, k = a.hidden, a.inter, a.experts, a.topk
    e_local = E // W
    Ts = [int(x) for x in a.tokens.split(",")]
    epg = EPGroup(ps, H, k, E, max(Ts))
    g = torch.Generator(device=dev).manual_seed(rank)
    w13 = (torch.randn(e_local, 2 * I, H, device=dev, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(e_local, H, I, device=dev, generator=g) * 0.02).bfloat16()
    CALLS = 10

    def timeit(fn, n=10):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(CALLS):
                fn()
        ts = []
        for _ in range(n):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / CALLS * 1e3)
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del gr
        return float(t)

    for T in Ts:
        h = (torch.randn(T, H, device=dev, generator=g) * 0.5).bfloat16()
        ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
        w = torch.rand(T, k, device=dev, generator=g)
        out = torch.empty_like(h)
        e0 = rank * e_local

        def copy_fn(hr, ir, wr, o):
            o.copy_(hr)

        def expert_fn(hr, ir, wr, o):
            moe_ops.fused_experts(hr, w13, w2, ir, wr, "silu", e0, out=o)

        row = {"T_per_rank": T}
        row["exchange_only"] = timeit(lambda: epg.moe(h, ids, w, copy_fn, out=out, tokens_bound=T))
        row["ep_layer"] = timeit(lambda: epg.moe(h, ids, w, expert_fn, out=out, tokens_bound=T))
        # the same routed work without an exchange: T tokens whose experts are all local
        ids_loc = (ids % e_local + e0).to(torch.int32)
        row["local_experts"] = timeit(lambda: moe_ops.fused_experts(h, w13, w2, ids_loc, w, "silu", e0, out=out))
        if rank == 0:
            print("ep " + " ".join(f"{k_}={v:.1f}" if isinstance(v, float) else f"{k_}={v}" for k_, v in row.items())
                  + f" world={W} status={epg.status()}", flush=True)
    epg.close()
    pdist.destroy(hard_exit_on_hang=True)


if __name__ == "__main__":
    main()
