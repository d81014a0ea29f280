"""Fused tensor-parallel reduction: all-reduce over NVLink peer memory + residual add + RMSNorm in
one kernel (`csrc/comm.cu`), used after every row-parallel GEMM.

The row-parallel GEMM writes its partial sums straight into this rank's symmetric `partial` buffer
(`partial_out(T)` hands out the view for the current call), then `reduce_residual_norm` launches the
kernel.  Two buffers alternate between calls; every forward pass issues an even number of calls (two per
layer), so the buffer a call site uses is the same on every CUDA-graph replay.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _count
from ..ops._native import check, f32, kernels, ptr, stream
from . import dist as pdist
from .symm import SymmetricRegion


def _ptr_array(vals):
    arr = (ctypes.c_void_p * len(vals))()
    for i, v in enumerate(vals):
        arr[i] = v
    return arr


class FusedTP:
    ONE_SHOT_BYTES = 512 * 1024  # per-rank message below which every rank pulls all rows itself

    def __init__(self, pstate: Optional[pdist.ParallelState] = None, max_tokens: int = 16384, hidden: int = 8192,
                 ctas: int = 592, push: bool = True, push_tokens: Optional[int] = 1024):
        ps = pstate or pdist.state()
        assert ps.device.type == "cuda" and 1 < ps.tp_size <= 8
        self.ps = ps
        self.world, self.rank = ps.tp_size, ps.tp_rank
        self.max_tokens, self.hidden = max_tokens, hidden
        self.ctas = ctas
        row_bytes = hidden * 2
        self.buf_bytes = ((max_tokens * row_bytes + 255) // 256) * 256
        self.off_partial = [0, self.buf_bytes]
        self.off_sums = [2 * self.buf_bytes, 3 * self.buf_bytes]
        self.off_ready = 4 * self.buf_bytes
        self.off_rowflag = self.off_ready + 256
        self.max_chunks = max_tokens // self.world + 2   # chunk flags per owner rank (a chunk is >= 1 row)
        end_flags = self.off_rowflag + ((self.world * self.max_chunks * 4 + 255) // 256) * 256
        # pushed mode: gather slots [parity][source rank][max_tokens, hidden] + column counters [parity][source][blocks]
        self.max_mb = (max_tokens + 127) // 128
        self.push_tokens = min(max_tokens, push_tokens if push_tokens is not None else max_tokens)
        self.off_gather = [end_flags, end_flags + self.world * self.buf_bytes] if push else None
        cnt_bytes = ((self.world * self.max_mb * 4 + 255) // 256) * 256
        self.off_cnt = [end_flags + 2 * self.world * self.buf_bytes + i * cnt_bytes for i in range(2)] if push else None
        total = end_flags + (2 * self.world * self.buf_bytes + 2 * cnt_bytes if push else 0)
        self.push = bool(push)
        group = ps.cpu_group if ps.cpu_group is not None else ps.tp_group
        self.region = SymmetricRegion(total, self.rank, self.world, group=ps.tp_group if ps.dp_size > 1 else group,
                                      device=ps.device)
        self.local = torch.zeros(8, dtype=torch.int32, device=ps.device)  # [epoch, arrive, status, pad, push_epoch0, push_epoch1]
        self.parity = 0
        self.calls = 0
        self._tabs = {}
        self.force_one_shot = None  # experiments: 0 / 1 overrides the size rule

    def close(self):
        self._tabs = {}
        self.region.close()

    # ---- buffers ----
    def partial_out(self, T: int, H: int) -> torch.Tensor:
        """Where the row-parallel GEMM of the next call must write its [T, H] partial sums."""
        assert T <= self.max_tokens and H == self.hidden
        return self.region.tensor(self.off_partial[self.parity], (T, H), torch.bfloat16)

    def prefers(self, T: int, H: int) -> bool:
        """Measured: with 4 or more ranks NCCL + the norm kernel wins above about 64 MB per rank (455 vs 534 us at
        134 MB on 4 GPUs); below that, and always with 2 ranks, the fused kernel is faster."""
        return self.world == 2 or T * H * 2 <= (64 << 20)

    def owns(self, partial) -> bool:
        """True if `partial` is the buffer handed out by `partial_out` for the coming call."""
        return partial.is_cuda and partial.data_ptr() == self.region.local_ptr + self.off_partial[self.parity]

    def _tables(self, par):
        t = self._tabs.get(par)
        if t is None:
            r = self.region
            base = self.local.data_ptr()
            t = self._tabs[par] = dict(
                partial=_ptr_array([r.ptrs[q] + self.off_partial[par] for q in range(self.world)]),
                sums=_ptr_array([r.ptrs[q] + self.off_sums[par] for q in range(self.world)]),
                ready=_ptr_array([r.ptrs[q] + self.off_ready for q in range(self.world)]),
                rowflag=_ptr_array([r.ptrs[q] + self.off_rowflag for q in range(self.world)]),
                epoch=_ptr_array([base]), arrive=_ptr_array([base + 4]), status=ctypes.c_void_p(base + 8))
        return t

    def _one_shot(self, T, H) -> int:
        # one-shot: every rank pulls all peers' rows, (world - 1) x the message inbound and no second phase;
        # two-shot: 2 (world - 1) / world x inbound plus a flag round.  With two ranks one-shot never moves more.
        if self.force_one_shot is not None:
            return self.force_one_shot
        return 1 if (self.world == 2 or T * H * 2 * (self.world - 1) <= 4 * self.ONE_SHOT_BYTES) else 0

    # ---- pushed mode: the GEMM stores its tiles into every rank's gather slot and counts columns ----
    def can_push(self, T: int, H: int) -> bool:
        return self.push and H == self.hidden and T <= self.push_tokens and H % 32 == 0 and self._one_shot(T, H) == 1

    def gemm_push(self, a, w, bias=None):
        """Row-parallel GEMM whose epilogue writes the partial sums of this rank into all ranks' gather slots
        (peer stores, tile by tile while the other tiles still compute).  Follow with reduce_pushed()."""
        from .. import ops

        par = self.parity
        key = ("push", par)
        t = self._tabs.get(key)
        if t is None:
            r = self.region
            slot = self.rank * self.buf_bytes
            t = self._tabs[key] = (_ptr_array([r.ptrs[q] + self.off_gather[par] + slot for q in range(self.world)]),
                                   _ptr_array([r.ptrs[q] + self.off_cnt[par] for q in range(self.world)]))
        check(kernels().llb_gemm_set_push(t[0], t[1], ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                          ctypes.c_int(self.max_mb)), "gemm_set_push")
        T, N = a.shape[0], w.shape[0]
        # `out` is only a shape / stride carrier: the kernel stores through the push pointers
        dummy = self.region.tensor(self.off_gather[par] + self.rank * self.buf_bytes, (T, N), torch.bfloat16)
        ops.gemm(a, w, bias=bias, out=dummy)
        return T, N

    def reduce_pushed(self, T, H, residual, norm_w, eps, w_offset=0.0):
        out = torch.empty((T, H), dtype=torch.bfloat16, device=residual.device)
        par = self.parity
        key = ("pushed", par)
        t = self._tabs.get(key)
        base = self.local.data_ptr()
        if t is None:
            r = self.region
            t = self._tabs[key] = dict(
                partial=_ptr_array([r.local_ptr + self.off_gather[par] + q * self.buf_bytes for q in range(self.world)]),
                cnt=_ptr_array([r.local_ptr + self.off_cnt[par]]), pepoch=_ptr_array([base + 16 + 4 * par]))
        tb = self._tables(par)
        check(kernels().llb_tp_reduce_norm(t["partial"], tb["sums"], tb["ready"], tb["rowflag"],
                                           _ptr_array([residual.data_ptr()]), _ptr_array([out.data_ptr()]), ptr(norm_w),
                                           tb["epoch"], tb["arrive"], tb["status"], ctypes.c_int(self.rank),
                                           ctypes.c_int(self.world), ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H),
                                           f32(eps), f32(w_offset), ctypes.c_int(2), ctypes.c_int(1),
                                           ctypes.c_int(min(self.ctas, max(T, 1))), ctypes.c_int(self.max_chunks),
                                           t["cnt"], t["pepoch"], ctypes.c_int(self.max_mb), stream()), "tp_reduce_pushed")
        _count()
        self.parity ^= 1
        self.calls += 1
        return out

    def _launch(self, T, H, residual, out, norm_w, eps, w_offset, do_norm):
        t = self._tables(self.parity)
        check(kernels().llb_tp_reduce_norm(t["partial"], t["sums"], t["ready"], t["rowflag"],
                                           _ptr_array([residual.data_ptr() if residual is not None else 0]),
                                           _ptr_array([out.data_ptr()]), ptr(norm_w), t["epoch"], t["arrive"],
                                           t["status"], ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                           ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H), f32(eps), f32(w_offset),
                                           ctypes.c_int(self._one_shot(T, H)), ctypes.c_int(do_norm),
                                           ctypes.c_int(min(self.ctas, max(T, 1))), ctypes.c_int(self.max_chunks),
                                           None, None, ctypes.c_int(0), stream()), "tp_reduce_norm")
        _count()
        self.parity ^= 1
        self.calls += 1

    def reduce_residual_norm(self, partial, residual, norm_w, eps, w_offset=0.0):
        """`partial` must be the tensor handed out by `partial_out` for this call."""
        T, H = partial.shape
        assert partial.data_ptr() == self.region.local_ptr + self.off_partial[self.parity], \
            "the row-parallel GEMM must write into FusedTP.partial_out()"
        out = torch.empty((T, H), dtype=torch.bfloat16, device=partial.device)
        self._launch(T, H, residual, out, norm_w, eps, w_offset, 1)
        return out

    def tpsp_reduce(self, partial, residual, norm_w, eps, w_offset=0.0):
        """Token-sharded variant (the reference's tpsp mix mode, lightllm/common/basemodel/layer_infer/template/
        transformer_layer_infer_template.py tpsp_* paths: reduce-scatter, norm on the shard, all-gather) as ONE
        kernel: each rank reduces the rows it owns (row % world == rank) from the peers' partial buffers, adds
        its shard of the residual stream, normalises, and stores the normalised rows into every rank's gather
        buffer.  Only the owned rows of `residual` are kept up to date.  Returns the complete normalised [T, H]
        activations as a view of a symmetric buffer that stays valid until the call after the next one."""
        T, H = partial.shape
        assert partial.data_ptr() == self.region.local_ptr + self.off_partial[self.parity]
        par = self.parity
        out = self.region.tensor(self.off_sums[par], (T, H), torch.bfloat16)
        t = self._tables(par)
        rows = (T + self.world - 1) // self.world
        check(kernels().llb_tp_reduce_norm(t["partial"], t["sums"], t["ready"], t["rowflag"],
                                           _ptr_array([residual.data_ptr()]), _ptr_array([out.data_ptr()]), ptr(norm_w),
                                           t["epoch"], t["arrive"], t["status"], ctypes.c_int(self.rank),
                                           ctypes.c_int(self.world), ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H),
                                           f32(eps), f32(w_offset), ctypes.c_int(3), ctypes.c_int(1),
                                           ctypes.c_int(min(self.ctas, max(rows, 1))), ctypes.c_int(self.max_chunks),
                                           None, None, ctypes.c_int(0), stream()), "tp_tpsp_reduce")
        _count()
        self.parity ^= 1
        self.calls += 1
        return out

    def skip(self):
        """A reduction of this forward pass went another way (the last layer has no following norm): keep the
        buffer alternation in step, so that every pass starts on the same buffer (CUDA-graph replays reuse the
        captured addresses and two consecutive calls must never share a buffer)."""
        self.parity ^= 1

    def check(self):
        """Raise if a bounded wait of the kernel ran out (a peer did not show up within a second)."""
        st = self.status()
        if st != 0:
            raise RuntimeError(f"fused tensor-parallel reduction timed out waiting for a peer (code {st}); "
                               "restart with --disable_symm_mem_allreduce to fall back to NCCL")

    def status(self) -> int:
        return int(self.local[2].item())

    def self_test(self, T: int = 24) -> bool:
        """Start-up probe: two small reductions (both buffer parities) through the fused kernel against NCCL + torch
        on the same numbers; every rank learns whether ALL ranks agreed, so they take the same decision about
        falling back.  A peer that does not show up ends the kernel's bounded wait with an error status, which
        counts as a failure.  Reference: lightllm/utils/dist_check_utils.py (2-GPU capability check before the
        custom all-reduce paths are enabled)."""
        import torch.distributed as dist

        dev, H = self.ps.device, self.hidden
        T = min(T, self.max_tokens)
        ok = True
        try:
            for k in range(2):
                g = torch.Generator(device=dev).manual_seed(4321 + 17 * k + self.rank)
                mine = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
                gs = torch.Generator(device=dev).manual_seed(99 + k)           # the same on every rank
                residual = torch.randn(T, H, generator=gs, device=dev).to(torch.bfloat16)
                norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
                total = mine.float()
                dist.all_reduce(total, group=self.ps.tp_group)
                want_res = residual.float() + total
                want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + 1e-6)
                partial = self.partial_out(T, H)
                partial.copy_(mine)
                res = residual.clone()
                got = self.reduce_residual_norm(partial, res, norm_w, 1e-6)
                torch.cuda.synchronize(dev)
                scale = max(want_res.abs().max().item(), 1.0)
                ok = ok and self.status() == 0 and \
                    (res.float() - want_res).abs().max().item() < 0.05 * scale and \
                    (got.float() - want).abs().max().item() < 0.05 * max(want.abs().max().item(), 1.0)
        except Exception:
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.ps.tp_group)
        return bool(flag.item())
