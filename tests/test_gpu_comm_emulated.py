"""The fused all-reduce + residual + RMSNorm kernel, all ranks emulated on ONE GPU: a single cooperative
launch with gridDim.y = world, every "rank" a slice of the same device memory, peer pointers = local
pointers.  Checks both modes (one-shot pull, two-shot reduce-scatter + push) over several epochs (the
flags are never reset) against an fp32 reference."""
import ctypes

import pytest
import torch

from lightllm_b200.ops import reference as ref
from lightllm_b200.ops._native import kernels
from lightllm_b200.parallel.fused import _ptr_array

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("T,H,one_shot", [(5, 4096, 1), (48, 4096, 0), (33, 8192, 0), (7, 2048, 0), (256, 4096, 0)])
def test_tp_reduce_norm_emulated(dev, world, T, H, one_shot):
    torch.manual_seed(0)
    maxT = 512
    partial = [torch.zeros(2, maxT, H, dtype=BF, device=dev) for _ in range(world)]
    sums = [torch.zeros(2, maxT, H, dtype=BF, device=dev) for _ in range(world)]
    ready = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    max_chunks = maxT // world + 2
    rowflag = [torch.zeros(world * max_chunks, dtype=torch.int32, device=dev) for _ in range(world)]
    local = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    residual = [(torch.randn(T, H, device=dev)).to(BF) for _ in range(world)]
    residual = [residual[0].clone() for _ in range(world)]  # replicated stream
    want_res = residual[0].float().clone()
    ctas = min(16, T)
    for call in range(4):
        par = call & 1
        parts = [(torch.randn(T, H, device=dev) * 0.5).to(BF) for _ in range(world)]
        for r in range(world):
            partial[r][par, :T] = parts[r]
        out = [torch.empty(T, H, dtype=BF, device=dev) for _ in range(world)]
        tab = lambda ts, sel: _ptr_array([sel(ts[q]) for _ in range(world) for q in range(world)])
        rc = kernels().llb_tp_reduce_norm(
            tab(partial, lambda t: t[par].data_ptr()), tab(sums, lambda t: t[par].data_ptr()),
            tab(ready, lambda t: t.data_ptr()), tab(rowflag, lambda t: t.data_ptr()),
            _ptr_array([t.data_ptr() for t in residual]), _ptr_array([t.data_ptr() for t in out]),
            ctypes.c_void_p(w.data_ptr()), _ptr_array([t.data_ptr() for t in local]),
            _ptr_array([t.data_ptr() + 4 for t in local]), ctypes.c_void_p(status.data_ptr()), ctypes.c_int(0),
            ctypes.c_int(world), ctypes.c_int(world), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_float(1e-5),
            ctypes.c_float(0.0), ctypes.c_int(one_shot), ctypes.c_int(1), ctypes.c_int(ctas), ctypes.c_int(max_chunks), None, None,
            ctypes.c_int(0),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a bounded wait ran out"
        total = sum(p.float() for p in parts)
        if not one_shot:
            total = total.to(BF).float()  # the pushed sums are bf16
        want_res = (want_res + total).to(BF).float()
        want_out = ref.rmsnorm(want_res.to(BF), w, 1e-5)
        for r in range(world):
            assert (residual[r].float() - want_res).abs().max().item() < 6e-2
            assert (out[r].float() - want_out.float()).abs().max().item() < 6e-2
            assert int(local[r][0].item()) == call + 1  # epoch advanced exactly once


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("T,N,K,bn", [(200, 1024, 2048, b) for b in (2002, 2004, 2008, 3002, 3004, 3008)] +
                         [(256, 4096, 2048, b) for b in (2002, 2004, 3002, 3004)])
def test_split_k_gemm_push_then_pushed_reduce_emulated(dev, world, T, N, K, bn):
    """The split-K kernels' push epilogue (finished units stored into every rank's slot, columns counted per
    128-row block) feeds the pushed reduction like the tile kernels' does."""
    test_gemm_push_then_pushed_reduce_emulated(dev, world, T, N, K, bn)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("T,N,K", [(200, 1024, 512), (256, 4096, 2048), (37, 2048, 4096), (700, 1024, 1024)])
def test_gemm_push_then_pushed_reduce_emulated(dev, world, T, N, K, bn=0):
    """GEMM epilogue in push mode (tiles stored into every rank's gather slot + column counters) followed by the
    reduce kernel in pushed mode; the ranks are slices of one GPU, run over three rounds without resetting."""
    from lightllm_b200 import ops

    torch.manual_seed(1)
    max_mb = (T + 127) // 128 + 1
    gather = [torch.zeros(world, T, N, dtype=BF, device=dev) for _ in range(world)]     # [dst rank][src rank]
    cnt = [torch.zeros(world * max_mb, dtype=torch.int32, device=dev) for _ in range(world)]
    local = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    dummy_tab = _ptr_array([0] * (world * world))
    norm_w = (torch.randn(N, device=dev) * 0.1 + 1).to(BF)
    residual = [torch.zeros(T, N, dtype=BF, device=dev) for _ in range(world)]
    want_res = torch.zeros(T, N, device=dev)
    for rnd in range(3):
        acts = [(torch.randn(T, K, device=dev) * 0.5).to(BF) for _ in range(world)]
        ws = [(torch.randn(N, K, device=dev) * 0.05).to(BF) for _ in range(world)]
        for r in range(world):   # rank r's GEMM pushes into slot r of every rank
            rc = kernels().llb_gemm_set_push(_ptr_array([gather[q][r].data_ptr() for q in range(world)]),
                                             _ptr_array([cnt[q].data_ptr() for q in range(world)]), ctypes.c_int(r),
                                             ctypes.c_int(world), ctypes.c_int(max_mb))
            assert rc == 0
            ops.gemm(acts[r], ws[r], out=gather[r][r], bn=bn)
        out = [torch.empty(T, N, dtype=BF, device=dev) for _ in range(world)]
        rc = kernels().llb_tp_reduce_norm(
            _ptr_array([gather[r][q].data_ptr() for r in range(world) for q in range(world)]), dummy_tab, dummy_tab,
            dummy_tab, _ptr_array([t.data_ptr() for t in residual]), _ptr_array([t.data_ptr() for t in out]),
            ctypes.c_void_p(norm_w.data_ptr()), _ptr_array([t.data_ptr() for t in local]),
            _ptr_array([t.data_ptr() + 4 for t in local]), ctypes.c_void_p(status.data_ptr()), ctypes.c_int(0),
            ctypes.c_int(world), ctypes.c_int(world), ctypes.c_int(T), ctypes.c_int(N), ctypes.c_float(1e-5),
            ctypes.c_float(0.0), ctypes.c_int(2), ctypes.c_int(1), ctypes.c_int(min(16, T)), ctypes.c_int(4),
            _ptr_array([t.data_ptr() for t in cnt]), _ptr_array([t.data_ptr() + 16 for t in local]),
            ctypes.c_int(max_mb), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a bounded wait ran out"
        assert int(ops.gemm_status(dev).item()) == 0
        total = sum((a.float() @ w.float().t()).to(BF).float() for a, w in zip(acts, ws))
        want_res = (want_res + total).to(BF).float()
        want_out = ref.rmsnorm(want_res.to(BF), norm_w, 1e-5).float()
        scale = want_res.abs().max().item()
        for r in range(world):
            assert (residual[r].float() - want_res).abs().max().item() < 2e-2 * scale + 5e-2
            assert (out[r].float() - want_out).abs().max().item() < 8e-2
            assert int(cnt[r][0].item()) == (rnd + 1) * N


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("T,H", [(5, 4096), (48, 4096), (33, 8192), (256, 2048), (1, 4096)])
def test_tpsp_reduce_emulated(dev, world, T, H):
    """Token-sharded mode: each rank reduces + normalises the rows it owns and pushes them to every rank's
    gather buffer; only the owned rows of each rank's residual are kept up to date."""
    torch.manual_seed(2)
    maxT = 512
    partial = [torch.zeros(2, maxT, H, dtype=BF, device=dev) for _ in range(world)]
    sums = [torch.zeros(2, maxT, H, dtype=BF, device=dev) for _ in range(world)]
    ready = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    max_chunks = maxT // world + 2
    rowflag = [torch.zeros(world * max_chunks, dtype=torch.int32, device=dev) for _ in range(world)]
    local = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    res0 = torch.randn(T, H, device=dev).to(BF)
    residual = [res0.clone() for _ in range(world)]
    want_res = res0.float().clone()
    ctas = min(16, max((T + world - 1) // world, 1))
    for call in range(4):
        par = call & 1
        parts = [(torch.randn(T, H, device=dev) * 0.5).to(BF) for _ in range(world)]
        for r in range(world):
            partial[r][par, :T] = parts[r]
        tab = lambda ts, sel: _ptr_array([sel(ts[q]) for _ in range(world) for q in range(world)])
        rc = kernels().llb_tp_reduce_norm(
            tab(partial, lambda t: t[par].data_ptr()), tab(sums, lambda t: t[par].data_ptr()),
            tab(ready, lambda t: t.data_ptr()), tab(rowflag, lambda t: t.data_ptr()),
            _ptr_array([t.data_ptr() for t in residual]), _ptr_array([s[par].data_ptr() for s in sums]),
            ctypes.c_void_p(w.data_ptr()), _ptr_array([t.data_ptr() for t in local]),
            _ptr_array([t.data_ptr() + 4 for t in local]), ctypes.c_void_p(status.data_ptr()), ctypes.c_int(0),
            ctypes.c_int(world), ctypes.c_int(world), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_float(1e-5),
            ctypes.c_float(0.0), ctypes.c_int(3), ctypes.c_int(1), ctypes.c_int(ctas), ctypes.c_int(max_chunks),
            None, None, ctypes.c_int(0), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a bounded wait ran out"
        want_res = (want_res + sum(p.float() for p in parts)).to(BF).float()
        want_out = ref.rmsnorm(want_res.to(BF), w, 1e-5).float()
        for r in range(world):
            if r < T:
                own = torch.arange(r, T, world, device=dev)
                assert (residual[r][own].float() - want_res[own]).abs().max().item() < 6e-2
            assert (sums[r][par, :T].float() - want_out).abs().max().item() < 6e-2
            assert int(local[r][0].item()) == call + 1


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("T,H", [(4096, 4096), (1000, 2048), (5, 4096), (2047, 8192)])
def test_copy_engine_reduce_emulated(dev, world, T, H):
    """The copy-engine reduction (flag exchange, slice pulls with cudaMemcpyAsync, local sum + residual + RMSNorm,
    pull of the normalised rows) with all ranks living on one GPU: the three phases of a call are run rank by
    rank, which is the order real ranks reach them in."""
    from lightllm_b200.parallel.ce import CopyEngineTP

    torch.manual_seed(5)
    maxT = 4096
    total = CopyEngineTP.layout(maxT, H)[1]
    regions = [torch.zeros(total, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [r.data_ptr() for r in regions]
    ranks = [CopyEngineTP(r, world, maxT, H, dev, ptrs, ptrs[r]) for r in range(world)]
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    res0 = torch.randn(T, H, device=dev).to(BF)
    residual = [res0.clone() for _ in range(world)]
    want_res = res0.float().clone()
    for call in range(4):
        parts = [(torch.randn(T, H, device=dev) * 0.5).to(BF) for _ in range(world)]
        for r in range(world):
            ranks[r].partial_out(T).copy_(parts[r])
        for mode in (1, 2):          # everybody announces, then everybody waits
            for r in range(world):
                ranks[r].phase_ready(mode)
        for r in range(world):
            ranks[r].phase_scatter_reduce(T, residual[r], w, 1e-5)
        for mode in (1, 2):
            for r in range(world):
                ranks[r].phase_normed(mode)
        outs = [ranks[r].phase_gather(T) for r in range(world)]
        torch.cuda.synchronize()
        assert all(rk.status() == 0 for rk in ranks), "a bounded wait ran out"
        want_res = (want_res + sum(p.float() for p in parts)).to(BF).float()
        want_out = ref.rmsnorm(want_res.to(BF), w, 1e-5).float()
        for r in range(world):
            lo, hi = ranks[r].rows_of(r, T)
            if hi > lo:
                assert (residual[r][lo:hi].float() - want_res[lo:hi]).abs().max().item() < 6e-2
            assert (outs[r].float() - want_out).abs().max().item() < 6e-2
