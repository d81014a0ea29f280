"""MoE kernels (routers, alignment, grouped tcgen05 GEMM, combine) against fp32 PyTorch restatements."""
import pytest
import torch

from lightllm_b200.ops import moe
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (77, 128, 8), (300, 8, 2), (64, 256, 8), (33, 60, 4)])
@pytest.mark.parametrize("renorm", [True, False])
def test_topk_softmax(dev, T, E, k, renorm):
    torch.manual_seed(0)
    logits = torch.randn(T, E, device=dev) * 2
    ids, w = moe.topk_softmax(logits, k, renorm, 1.0)
    rids, rw = moe.ref_topk_softmax(logits, k, renorm, 1.0)
    assert torch.equal(ids.sort(-1)[0], rids.sort(-1)[0])
    assert torch.allclose(w.sort(-1)[0], rw.sort(-1)[0], atol=1e-5, rtol=1e-4)
    ids2, w2 = moe.topk_softmax(logits.to(BF), k, renorm, 1.0)
    assert ids2.shape == (T, k)


@pytest.mark.parametrize("T", [1, 50, 257])
@pytest.mark.parametrize("with_bias", [True, False])
def test_grouped_topk_deepseek(dev, T, with_bias):
    torch.manual_seed(1)
    E, k, ng, tg = 256, 8, 8, 4
    logits = torch.randn(T, E, device=dev)
    bias = (torch.randn(E, device=dev) * 0.1) if with_bias else None
    ids, w = moe.grouped_topk(logits, bias, k, ng, tg, True, True, 2.5)
    rids, rw = moe.ref_grouped_topk(logits, bias, k, ng, tg, True, True, 2.5)
    assert torch.equal(ids.sort(-1)[0], rids.sort(-1)[0])
    assert torch.allclose(w.sort(-1)[0], rw.sort(-1)[0], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("T,E,k,H,I,e0,El", [(64, 8, 2, 512, 256, 0, 8), (200, 128, 8, 2048, 768, 0, 128),
                                             (1, 128, 8, 2048, 768, 0, 128), (300, 32, 4, 1024, 512, 8, 8)])
def test_fused_experts(dev, T, E, k, H, I, e0, El):
    torch.manual_seed(2)
    x = (torch.randn(T, H, device=dev) * 0.5).to(BF)
    g = (torch.randn(El, I, H, device=dev) * 0.05).to(BF)
    u = (torch.randn(El, I, H, device=dev) * 0.05).to(BF)
    w13 = ref.interleave_gate_up(g, u)
    w2 = (torch.randn(El, H, I, device=dev) * 0.05).to(BF)
    logits = torch.randn(T, E, device=dev)
    ids, w = moe.topk_softmax(logits, k, True, 1.0)
    got = moe.fused_experts(x, w13, w2, ids, w, "silu", e0)
    want = moe.ref_fused_experts(x, w13, w2, ids, w, "silu", e0)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2 * want.float().abs().max().item() + 2e-2, err
    # accumulate on top of a shared-expert output
    base = torch.randn(T, H, device=dev).to(BF)
    acc = base.clone()
    moe.fused_experts(x, w13, w2, ids, w, "silu", e0, out=acc, accumulate=True)
    assert (acc.float() - (base.float() + want.float())).abs().max().item() < 6e-2


@pytest.mark.parametrize("T,k,E", [(1, 8, 128), (300, 8, 256), (5000, 4, 64)])
def test_count_remap_matches_cpu(dev, T, k, E):
    """Physical-id rewrite + hit counters of the redundant-expert path: the kernel against the torch restatement."""
    from lightllm_b200.engine.redundancy import physical_table

    g = torch.Generator().manual_seed(T)
    ids = torch.randint(-1, E, (T, k), generator=g, dtype=torch.int32)
    table = physical_table(E, 8, 3, [0, 1, E - 1, E // 2])
    cnt_ref = torch.zeros(E, dtype=torch.int32)
    want = moe.count_remap(ids, table, cnt_ref)
    cnt = torch.zeros(E, dtype=torch.int32, device=dev)
    got = moe.count_remap(ids.to(dev), table.to(dev), cnt)
    assert torch.equal(got.cpu(), want) and torch.equal(cnt.cpu(), cnt_ref)
    assert torch.equal(moe.count_remap(ids.to(dev), table.to(dev), None).cpu(), want)


@pytest.mark.parametrize("E,T,k", [(128, 300, 8), (384, 77, 6)])
def test_route_capture_scatter_matches_cpu(dev, E, T, k):
    """Routed-expert capture: the scatter kernel (8- and 16-bit ids) against the torch indexing restatement."""
    from lightllm_b200.common.route_capture import RouteCapture

    cfg = dict(num_hidden_layers=4, num_experts=E, num_experts_per_tok=k, decoder_sparse_step=1, mlp_only_layers=[1])
    g = torch.Generator().manual_seed(E)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    slots = torch.randperm(1000, generator=g)[:T].to(torch.int32)
    a, b = RouteCapture(cfg, 1000, "cpu"), RouteCapture(cfg, 1000, dev)
    for layer in (0, 2, 3, 1):           # layer 1 is dense: ignored
        a.capture(layer, ids + 0, slots)
        b.capture(layer, ids.to(dev), slots.to(dev))
        ids = (ids + 1) % E
    assert torch.equal(b.buf.cpu(), a.buf)
    pick = slots[:10]
    assert (b.extract(pick) == a.extract(pick)).all()
