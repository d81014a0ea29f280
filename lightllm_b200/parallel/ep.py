"""Expert-parallel token exchange for data-parallel attention (`--dp` equal to the world size, `--enable_ep_moe`).

Every rank runs attention on its own requests; in a MoE layer a token has to reach the ranks that own its
experts and the partial results have to come back.  `EPGroup.moe(h, ids, w, expert_fn, out)` does that:

* CUDA: `csrc/ep.cu` - the ranks write tokens straight into each other's receive buffers over NVLink peer
  memory (symmetric region mapped through CUDA IPC), run their experts over what they received, and pull the
  partial sums back with peer loads; counts, flags and offsets stay on the devices, no host round trip, fixed
  worst-case launch shapes.
* CPU / gloo (tests, fallback): all-gather of the padded token blocks, local experts over everything, all-reduce
  of the partial sums, own rows sliced out.

Reference: lightllm/common/basemodel/layer_weights/meta_weights/fused_moe/* (DeepEP dispatch / combine).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _count
from ..ops._native import check, kernels, ptr, stream
from . import dist as pdist


def _ptr_array(vals):
    arr = (ctypes.c_void_p * len(vals))()
    for i, v in enumerate(vals):
        arr[i] = v
    return arr


class EPGroup:
    def __init__(self, ps: pdist.ParallelState, hidden: int, top_k: int, num_experts: int, max_tokens: int,
                 max_recv: int = 0, ctas: int = 296):
        self.ps = ps
        self.world, self.rank = ps.world_size, ps.global_rank
        assert num_experts % self.world == 0, "experts must divide evenly over the expert-parallel ranks"
        self.e_local = num_experts // self.world
        self.hidden, self.k = hidden, top_k
        self.max_tokens = max_tokens
        self.max_recv = max_recv or self.world * max_tokens
        self.device = ps.device
        self.cuda = ps.device.type == "cuda"
        self.ctas = ctas
        if not self.cuda:
            return
        from .symm import SymmetricRegion

        H, k, R, W = hidden, top_k, self.max_recv, self.world
        al = lambda n: (n + 255) // 256 * 256  # noqa: E731
        self.off_h = 0
        self.off_out = al(R * H * 2)
        self.off_ids = self.off_out + al(R * H * 2)
        self.off_w = self.off_ids + al(R * k * 4)
        self.off_counts = self.off_w + al(R * k * 4)
        self.off_flags = self.off_counts + al(W * W * 4)
        total = self.off_flags + al(3 * W * 4)
        self.region = SymmetricRegion(total, self.rank, W, group=ps.cpu_group if ps.cpu_group is not None else None,
                                      device=self.device)
        r = self.region
        self.t_h = _ptr_array([r.ptrs[q] + self.off_h for q in range(W)])
        self.t_out = _ptr_array([r.ptrs[q] + self.off_out for q in range(W)])
        self.t_ids = _ptr_array([r.ptrs[q] + self.off_ids for q in range(W)])
        self.t_w = _ptr_array([r.ptrs[q] + self.off_w for q in range(W)])
        self.t_counts = _ptr_array([r.ptrs[q] + self.off_counts for q in range(W)])
        self.t_flags = _ptr_array([r.ptrs[q] + self.off_flags for q in range(W)])
        self.h_recv = r.tensor(self.off_h, (R, H), torch.bfloat16)
        self.out_recv = r.tensor(self.off_out, (R, H), torch.bfloat16)
        self.ids_recv = r.tensor(self.off_ids, (R, k), torch.int32)
        self.w_recv = r.tensor(self.off_w, (R, k), torch.float32)
        self.ids_recv.fill_(-1)
        dev = self.device
        self.dest_mask = torch.zeros(max_tokens, dtype=torch.uint8, device=dev)
        self.slot = torch.zeros((max_tokens, 8), dtype=torch.int32, device=dev)
        self.where = torch.zeros((max_tokens, 8), dtype=torch.int32, device=dev)
        self.local = torch.zeros(8, dtype=torch.int32, device=dev)  # [arrive_push, arrive_combine, status, epoch, recv_total]
        torch.cuda.synchronize(dev)
        if ps.cpu_group is not None:
            dist.barrier(group=ps.cpu_group)  # every rank's buffers are initialised before the first round

    # ------------------------------------------------------------------
    def moe(self, h, ids, w, expert_fn, out=None, accumulate: bool = False, tokens_bound: int = 0):
        """out[t] (+)= sum over the token's experts, wherever they live.  `expert_fn(h_rows, ids_rows, w_rows,
        out_rows)` must add nothing for expert ids that are not local.

        `tokens_bound`: an upper bound on the number of tokens ANY rank brings to this exchange, the same value
        on every rank (0: the group's `max_tokens`).  The experts then run over world x tokens_bound receive rows
        instead of the worst case the buffers were sized for, which is what keeps a decode step (a few hundred
        tokens in all) from paying for a prompt-sized launch."""
        T = h.shape[0]
        if out is None:
            out = torch.empty_like(h)
            accumulate = False
        if self.world == 1:
            tmp = torch.empty_like(h)
            expert_fn(h, ids, w, tmp)
            return out.add_(tmp) if accumulate else out.copy_(tmp)
        if not self.cuda:
            return self._moe_gather_reduce(h, ids, w, expert_fn, out, accumulate)
        assert T <= self.max_tokens and h.is_contiguous() and ids.dtype == torch.int32 and w.dtype == torch.float32
        rows = self.max_recv
        if tokens_bound > 0:
            assert T <= tokens_bound, "tokens_bound must cover every rank's token count"
            rows = min(self.max_recv, self.world * tokens_bound)
        base = self.local.data_ptr()
        lib = kernels()
        check(lib.llb_ep_dispatch(self.t_h, self.t_ids, self.t_w, self.t_out, self.t_counts, self.t_flags,
                                  ctypes.c_int(self.rank), ctypes.c_int(self.world), ptr(h), ptr(ids), ptr(w),
                                  ctypes.c_int(T), ctypes.c_int(self.hidden), ctypes.c_int(self.k),
                                  ctypes.c_int(self.e_local), ctypes.c_int(rows), ptr(self.dest_mask),
                                  ptr(self.slot), ptr(self.where), ctypes.c_void_p(base), ctypes.c_void_p(base + 16),
                                  ctypes.c_void_p(base + 8), ctypes.c_void_p(base + 12),
                                  ctypes.c_int(min(self.ctas, max(T, 1))), stream()), "ep_dispatch")
        _count(3)
        expert_fn(self.h_recv[:rows], self.ids_recv[:rows], self.w_recv[:rows], self.out_recv[:rows])
        check(lib.llb_ep_combine(self.t_h, self.t_ids, self.t_w, self.t_out, self.t_counts, self.t_flags,
                                 ctypes.c_int(self.rank), ctypes.c_int(self.world), ptr(out), ctypes.c_int(T),
                                 ctypes.c_int(self.hidden), ptr(self.where), ctypes.c_int(1 if accumulate else 0),
                                 ctypes.c_void_p(base + 8), ctypes.c_void_p(base + 12), ctypes.c_void_p(base + 4),
                                 ctypes.c_int(min(self.ctas, max(T, 1))), stream()), "ep_combine")
        _count()
        return out

    def _moe_gather_reduce(self, h, ids, w, expert_fn, out, accumulate):
        g = self.ps.cpu_group if not self.cuda else None
        T = h.shape[0]
        counts = torch.zeros(self.world, dtype=torch.int64)
        mine = torch.tensor([T], dtype=torch.int64)
        dist.all_gather_into_tensor(counts, mine, group=g)
        mx = int(counts.max())
        pad = lambda x, fill: torch.cat([x, x.new_full((mx - T, *x.shape[1:]), fill)]) if mx > T else x  # noqa: E731
        H, k = self.hidden, self.k
        all_h = torch.empty((self.world * mx, H), dtype=h.dtype)
        all_i = torch.empty((self.world * mx, k), dtype=ids.dtype)
        all_w = torch.empty((self.world * mx, k), dtype=w.dtype)
        dist.all_gather_into_tensor(all_h, pad(h, 0).contiguous(), group=g)
        dist.all_gather_into_tensor(all_i, pad(ids, -1).contiguous(), group=g)
        dist.all_gather_into_tensor(all_w, pad(w, 0).contiguous(), group=g)
        part = torch.zeros((self.world * mx, H), dtype=torch.float32)
        if mx:
            tmp = torch.zeros((self.world * mx, H), dtype=h.dtype)
            expert_fn(all_h, all_i, all_w, tmp)
            part = tmp.float()
        dist.all_reduce(part, group=g)
        own = part[self.rank * mx:self.rank * mx + T].to(h.dtype)
        return out.add_(own) if accumulate else out.copy_(own)

    def status(self) -> int:
        return int(self.local[2].item()) if self.cuda else 0

    def check(self):
        st = self.status()
        if st != 0:
            raise RuntimeError(f"expert-parallel exchange failed (code {st}): a peer did not show up within a second "
                               "or a receive buffer overflowed")

    def close(self):
        if self.cuda:
            self.region.close()
