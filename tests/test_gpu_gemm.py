"""tcgen05 bf16 GEMM and its epilogues against fp32 matmul."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _check(got, want, K):
    err = (got.float() - want.float()).abs().max().item()
    tol = 1e-2 * want.abs().max().item() + 1e-2  # bf16 output rounding (2^-8 relative) plus accumulation order
    assert err < tol, f"max abs err {err} (tol {tol})"
    assert int(ops.gemm_status(got.device).item()) == 0, "a bounded wait inside the GEMM timed out"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (1, 256, 128), (77, 512, 4096), (256, 6144, 4096),
                                   (300, 1024, 1000), (2048, 4096, 14336), (129, 16032, 512), (4096, 1280, 8192)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_store(dev, M, N, K, bn):
    torch.manual_seed(0)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    got = ops.gemm(a, w, bn=bn)
    _check(got, a.float() @ w.float().t(), K)


def test_gemm_epilogues(dev):
    torch.manual_seed(1)
    M, N, K = 200, 1024, 768
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    bias = torch.randn(N, device=dev).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    acc = a.float() @ w.float().t()
    _check(ops.gemm(a, w, bias=bias), acc + bias.float(), K)
    _check(ops.gemm(a, w, epi="residual", residual=res), acc + res.float(), K)
    r2 = res.clone()
    ops.gemm(a, w, epi="residual", residual=r2, out=r2)  # in place on the residual stream
    _check(r2, acc + res.float(), K)
    f = ops.gemm(a, w, epi="f32")
    assert f.dtype == torch.float32
    assert (f - acc).abs().max().item() < 1e-2
    # gated (SwiGLU): interleaved weights
    I = 512
    g = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    u = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    wi = ref.interleave_gate_up(g, u)
    want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
    for bn in (64, 128, 256):
        _check(ops.gemm(a, wi, epi="gated_silu", bn=bn), want, K)
    want_g = torch.nn.functional.gelu(a.float() @ g.float().t(), approximate="tanh") * (a.float() @ u.float().t())
    _check(ops.gemm(a, wi, epi="gated_gelu"), want_g, K)


def test_gemm_strided_a_and_tail_n(dev):
    torch.manual_seed(2)
    M, K, N = 150, 512, 264  # N not a multiple of 32
    big = (torch.randn(M, K + 256, device=dev) * 0.5).to(BF)
    a = big[:, :K]  # row stride K+256
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    _check(ops.gemm(a, w), a.float() @ w.float().t(), K)


@pytest.mark.parametrize("M,N,K", [(256, 4096, 4096), (256, 6144, 4096), (256, 28672, 4096), (256, 4096, 14336),
                                   (1, 4096, 4096), (17, 1024, 512), (300, 768, 8192), (2000, 2048, 1024)])
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_gemm_stream_k(dev, M, N, K, bn):
    """Tiles split across CTAs along K and fixed up by the last arriver; run twice to check that the
    arrival counters are left clean."""
    torch.manual_seed(3)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    want = a.float() @ w.float().t()
    for _ in range(2):
        _check(ops.gemm(a, w, bn=bn, stream_k=1), want, K)
    res = torch.randn(M, N, device=dev).to(BF)
    _check(ops.gemm(a, w, epi="residual", residual=res, bn=bn, stream_k=1), want + res.float(), K)


def test_gemm_stream_k_gated(dev):
    torch.manual_seed(4)
    M, I, K = 256, 1792, 4096
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    g = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    u = (torch.randn(I, K, device=dev) * 0.1).to(BF)
    wi = ref.interleave_gate_up(g, u)
    want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
    _check(ops.gemm(a, wi, epi="gated_silu", stream_k=1), want, K)
    _check(ops.gemm(a, wi, epi="gated_silu", stream_k=-1), want, K)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("M,N,K", [(256, 1024, 4096), (77, 512, 512), (1000, 2048, 1024)])
def test_gemm_preswizzled_tiled_weight(dev, bn, M, N, K):
    """W stored as 128B-swizzled 128 x 64 tiles and fetched with untiled bulk copies."""
    torch.manual_seed(7)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    _check(ops.gemm(a, ops.TiledWeight(w, swizzle=True), bn=bn), a.float() @ w.float().t(), K)


# Per-rank shapes of Llama-3-8B and Llama-3-70B under 8-way tensor parallelism (qkv, o_proj, gate_up, down, lm_head):
# narrow K and N that are not multiples of the widest tile, at decode and prefill row counts, automatic tile plan.
@pytest.mark.parametrize("M", [32, 256, 3000])
@pytest.mark.parametrize("N,K,epi", [(768, 4096, "store"), (4096, 512, "store"), (3584, 4096, "gated_silu"),
                                     (4096, 1792, "store"), (16032, 4096, "f32"), (1280, 8192, "store"),
                                     (8192, 1024, "store"), (7168, 8192, "gated_silu"), (8192, 3584, "store")])
def test_gemm_tp8_shard_shapes(dev, M, N, K, epi):
    torch.manual_seed(4)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.05).to(BF)
    acc = a.float() @ w.float().t()
    if epi == "gated_silu":
        wg, wu = w[: N // 2], w[N // 2:]
        want = torch.nn.functional.silu(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
        _check(ops.gemm(a, ref.interleave_gate_up(wg, wu), epi=epi), want, K)
    elif epi == "f32":
        got = ops.gemm(a, w, epi="f32")
        assert (got - acc).abs().max().item() < 1e-2 * acc.abs().max().item() + 1e-2
    else:
        _check(ops.gemm(a, w), acc, K)
