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
            ctypes.c_float(0.0), ctypes.c_int(one_shot), ctypes.c_int(1), ctypes.c_int(ctas), ctypes.c_int(max_chunks),
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
