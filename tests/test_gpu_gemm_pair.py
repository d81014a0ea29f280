"""CTA-pair (cta_group::2, 256x256 tiles) variant of the tcgen05 GEMM against fp32 matmul."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _check(got, want):
    err = (got.float() - want.float()).abs().max().item()
    tol = 1e-2 * want.abs().max().item() + 1e-2
    assert int(ops.gemm_status(got.device).item()) == 0, "a bounded wait inside the GEMM timed out"
    assert err < tol, f"max abs err {err} (tol {tol})"


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 256, 512), (512, 1024, 4096), (300, 768, 1000),
                                   (4096, 6144, 4096), (1000, 16032, 512), (16384, 4096, 4096)])
def test_pair_store(dev, M, N, K):
    torch.manual_seed(0)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    _check(ops.gemm(a, w, bn=512), a.float() @ w.float().t())


def test_pair_epilogues(dev):
    torch.manual_seed(1)
    M, N, K = 1500, 2048, 1024
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    acc = a.float() @ w.float().t()
    r2 = res.clone()
    ops.gemm(a, w, epi="residual", residual=r2, out=r2, bn=512)
    _check(r2, acc + res.float())
    f = ops.gemm(a, w, epi="f32", bn=512)
    assert (f - acc).abs().max().item() < 1e-2
    I = 1024
    g = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    u = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
    _check(ops.gemm(a, ref.interleave_gate_up(g, u), epi="gated_silu", bn=512), want)
