"""Times the fused NVLink all-reduce + residual + RMSNorm kernel against NCCL all-reduce followed by the
standalone add+RMSNorm kernel, over message sizes, grid sizes and both algorithms.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29621 -m lightllm_b200.benchmark.comm_bench

CUDA events on the launching stream, 3 warm-up and 30 timed calls back to back, max over ranks.  Both sides
include their host launch cost (two launches for the NCCL side, one for the fused kernel).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


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
