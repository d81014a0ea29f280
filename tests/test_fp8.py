"""Block-scaled fp8 (e4m3, 128 x 128 weight blocks, per-token-group activations): quantisers, the CPU arithmetic and
(on a GPU) the tcgen05 kernel against an fp32 reference of the same quantised operands."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import fp8
from lightllm_b200.ops import reference as ref

BF = torch.bfloat16


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def test_weight_and_activation_quant_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(300, 520) * 0.05
    fw = fp8.Fp8Weight.from_float(w)
    assert fw.scale.shape == (3, 5)
    assert _rel(fw.dequant(), w) < 0.07  # e4m3: 3 mantissa bits
    x = torch.randn(9, 520).to(BF)
    xq, xs = fp8.quant_act(x)
    assert xs.shape == (5, 9)
    assert _rel(fp8.dequant_act(xq, xs), x) < 0.07


def test_cpu_gemm_paths_match_dequantised_matmul():
    torch.manual_seed(1)
    x = (torch.randn(70, 384) * 0.5).to(BF)
    w = torch.randn(256, 384) * 0.05
    fw = fp8.Fp8Weight.from_float(w)
    got = ops.gemm(x, fw)
    want = x.float() @ w.t()
    assert _rel(got, want) < 0.06
    res = torch.randn(70, 256).to(BF)
    assert _rel(ops.gemm(x, fw, epi="residual", residual=res), want + res.float()) < 0.06
    g, u = fp8.Fp8Weight.from_float(w[:128]), fp8.Fp8Weight.from_float(w[128:])
    wi = fp8.interleave_gate_up_fp8(g, u)
    assert wi.ws_rows == 32 and wi.scale.shape == (8, 3)
    assert torch.equal(wi.dequant(), ref.interleave_gate_up(g.dequant(), u.dequant()))
    want_g = torch.nn.functional.silu(x.float() @ w[:128].t()) * (x.float() @ w[128:].t())
    assert _rel(ops.gemm(x, wi, epi="gated_silu"), want_g) < 0.08


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (1, 256, 512), (77, 512, 7168), (300, 4096, 512), (256, 2048, 2048),
                                   (1000, 1536, 1536), (130, 264, 400)])
def test_gpu_fp8_gemm_matches_fp32_of_quantised_operands(dev, M, N, K):
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = torch.randn(N, K, device=dev) * 0.05
    fw = fp8.Fp8Weight.from_float(w)
    xq, xs = fp8.quant_act(x)
    xq_ref, xs_ref = fp8.quant_act_reference(x)
    assert (xs - xs_ref).abs().max().item() <= 1e-6 * xs_ref.abs().max().item() + 1e-12
    assert (xq.float() - xq_ref.float()).abs().max().item() <= 32.0  # at most one e4m3 step at the top of the range
    want = fp8.dequant_act(xq, xs) @ fw.dequant().t()
    got = fp8.gemm_fp8_quantized(xq, xs, fw)
    assert _rel(got, want) < 6e-3, "bf16 rounding of the output only"
    res = torch.randn(M, N, device=dev).to(BF)
    got_r = fp8.gemm_fp8_quantized(xq, xs, fw, "residual", residual=res)
    assert _rel(got_r, want + res.float()) < 6e-3
    assert int(ops.gemm_status(dev).item()) == 0
    assert _rel(ops.gemm(x, fw), x.float() @ w.t()) < 0.06  # end to end against the unquantised product


@pytest.mark.gpu
def test_gpu_fp8_gated_and_grouped(dev):
    torch.manual_seed(5)
    M, I, K, E = 256, 512, 1024, 4
    x = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    xq, xs = fp8.quant_act(x)
    a = fp8.dequant_act(xq, xs)
    g = [fp8.Fp8Weight.from_float(torch.randn(I, K, device=dev) * 0.05) for _ in range(E)]
    u = [fp8.Fp8Weight.from_float(torch.randn(I, K, device=dev) * 0.05) for _ in range(E)]
    wi = [fp8.interleave_gate_up_fp8(g[e], u[e]) for e in range(E)]
    want0 = torch.nn.functional.silu(a @ g[0].dequant().t()) * (a @ u[0].dequant().t())
    assert _rel(fp8.gemm_fp8_quantized(xq, xs, wi[0], "gated_silu"), want0) < 8e-3
    stacked = fp8.stack_experts(wi)
    mbe = torch.tensor([2, -1], dtype=torch.int32, device=dev)
    got = fp8.gemm_fp8_quantized(xq, xs, stacked, "gated_silu", mblock_expert=mbe, n_per_expert=2 * I)
    want2 = torch.nn.functional.silu(a[:128] @ g[2].dequant().t()) * (a[:128] @ u[2].dequant().t())
    assert _rel(got[:128], want2) < 8e-3
    down = fp8.stack_experts([fp8.Fp8Weight.from_float(torch.randn(K, I, device=dev) * 0.05) for _ in range(E)])
    h = (torch.randn(M, I, device=dev) * 0.5).to(BF)
    hq, hs = fp8.quant_act(h)
    mbe2 = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    got_d = fp8.gemm_fp8_quantized(hq, hs, down, mblock_expert=mbe2, n_per_expert=K)
    hd = fp8.dequant_act(hq, hs)
    wd = down.dequant()
    assert _rel(got_d[:128], hd[:128] @ wd[3 * K:4 * K].t()) < 6e-3
    assert _rel(got_d[128:], hd[128:] @ wd[K:2 * K].t()) < 6e-3
    assert int(ops.gemm_status(dev).item()) == 0
