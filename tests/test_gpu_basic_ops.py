"""CUDA kernels of ops_basic.cu / sampling.cu against the fp32 PyTorch restatements."""
import math

import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def close(a, b, atol, rtol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"max abs err {err}"


@pytest.mark.parametrize("T,H", [(1, 256), (7, 4096), (33, 8192), (5, 7168), (3, 16384), (4, 576)])
def test_rmsnorm(dev, T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device=dev, dtype=BF)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    close(ops.rmsnorm(x, w, 1e-6), ref.rmsnorm(x, w, 1e-6), 2e-2)
    close(ops.rmsnorm(x, w, 1e-6, 1.0), ref.rmsnorm(x, w, 1e-6, 1.0), 4e-2)


@pytest.mark.parametrize("T,H", [(1, 4096), (19, 4096), (8, 8192)])
def test_add_rmsnorm(dev, T, H):
    torch.manual_seed(1)
    x = torch.randn(T, H, device=dev, dtype=BF)
    r = torch.randn(T, H, device=dev, dtype=BF)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    r2 = r.clone()
    want = ref.add_rmsnorm_(r2, x, w, 1e-5)
    got = ops.add_rmsnorm_(r, x, w, 1e-5)
    close(r, r2, 1e-2)
    close(got, want, 3e-2)


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_gated_act(dev, act):
    torch.manual_seed(2)
    x = torch.randn(37, 2 * 1792, device=dev, dtype=BF)
    close(ops.gated_act(x, act), ref.gated_act(x, act), 2e-2)


@pytest.mark.parametrize("D,Hq,Hkv,rot,qknorm", [(128, 32, 8, 128, False), (128, 4, 1, 128, True), (64, 8, 2, 64, False),
                                                 (128, 8, 8, 64, False), (256, 4, 2, 256, True)])
def test_rope_kv_scatter(dev, D, Hq, Hkv, rot, qknorm):
    torch.manual_seed(3)
    T, slots = 29, 101
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, dtype=BF)
    kv = torch.zeros(slots, 2 * Hkv, D, device=dev, dtype=BF)
    cos, sin = ref.build_rope_cache(512, rot, 1e4, None, device=dev)
    pos = torch.randint(0, 512, (T,), device=dev, dtype=torch.int32)
    slot = torch.randperm(slots, device=dev)[:T].to(torch.int32)
    qw = kw = None
    if qknorm:
        qw = (torch.randn(D, device=dev) * 0.1 + 1).to(BF)
        kw = (torch.randn(D, device=dev) * 0.1 + 1).to(BF)
    qkv2, kv2 = qkv.clone(), kv.clone()
    ref.rope_kv_scatter_(qkv2, kv2, cos, sin, pos, slot, Hq, Hkv, D, rot, qw, kw, 1e-6)
    ops.rope_kv_scatter_(qkv, kv, cos, sin, pos, slot, Hq, Hkv, D, rot, qw, kw, 1e-6)
    close(qkv[:, : Hq * D], qkv2[:, : Hq * D], 5e-2)
    close(kv, kv2, 5e-2)


def test_embedding(dev):
    torch.manual_seed(4)
    table = torch.randn(1000, 512, device=dev, dtype=BF)
    ids = torch.randint(0, 2000, (77,), device=dev)
    got = ops.embedding(ids, table, 500, 1500)
    want = ref.embedding(ids, table, 500, 1500)
    assert torch.equal(got, want)


def test_prologues_and_copy(dev):
    torch.manual_seed(5)
    max_req, max_len = 16, 64
    r2t = torch.zeros(max_req + 1, max_len, dtype=torch.int32, device=dev)
    nxt = torch.randint(0, 1000, (max_req + 1, 8), device=dev)
    b_req = torch.tensor([3, 7, 1], dtype=torch.int32, device=dev)
    b_len = torch.tensor([5, 9, 2], dtype=torch.int32, device=dev)
    slot = torch.tensor([100, 200, 300], dtype=torch.int32, device=dev)
    ids, pos = ops.decode_prologue(r2t, nxt, b_req, b_len, slot)
    assert ids.tolist() == nxt[b_req.long(), 0].tolist()
    assert pos.tolist() == [4, 8, 1]
    assert r2t[3, 4].item() == 100 and r2t[7, 8].item() == 200 and r2t[1, 1].item() == 300
    # prefill
    ready = torch.tensor([2, 0, 5], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, 3, 7, 9], dtype=torch.int32, device=dev)
    new = torch.arange(1000, 1009, dtype=torch.int32, device=dev)
    p, bo = ops.prefill_prologue(r2t, b_req, ready, cu, new, 9)
    assert p.tolist() == [2, 3, 4, 0, 1, 2, 3, 5, 6]
    assert bo.tolist() == [0, 0, 0, 1, 1, 1, 1, 2, 2]
    assert r2t[3, 2:5].tolist() == [1000, 1001, 1002] and r2t[1, 5:7].tolist() == [1007, 1008]
    # scatter next token
    sampled = torch.tensor([11, 22, 33], device=dev)
    has = torch.tensor([1, 0, 1], dtype=torch.uint8, device=dev)
    old7 = nxt[7, 0].item()
    ops.scatter_next_token_(nxt, sampled, b_req, has)
    assert nxt[3, 0].item() == 11 and nxt[7, 0].item() == old7 and nxt[1, 0].item() == 33
    # row copy
    src = torch.randn(50, 4, 64, device=dev, dtype=BF)
    dst = torch.zeros(20, 4, 64, device=dev, dtype=BF)
    si = torch.tensor([5, 6, 49], dtype=torch.int32, device=dev)
    di = torch.tensor([0, 19, 7], dtype=torch.int32, device=dev)
    ops.copy_rows(dst, src, di, si, 3)
    assert torch.equal(dst[0], src[5]) and torch.equal(dst[19], src[6]) and torch.equal(dst[7], src[49])
    host = torch.empty(3, 4, 64, dtype=BF).pin_memory()
    ops.copy_rows(host, src, None, si, 3)
    torch.cuda.synchronize()
    assert torch.equal(host, src[si.long()].cpu())


def test_sampler_greedy_and_logprob(dev):
    torch.manual_seed(6)
    B, V = 9, 32003
    logits = torch.randn(B, V, device=dev) * 3
    ids, lp = ops.sample(logits)
    want_ids, want_lp = ref.sample(logits)
    assert ids.tolist() == want_ids.tolist()
    close(lp, want_lp, 1e-3, 1e-3)
    some = torch.randint(0, V, (B,), device=dev)
    close(ops.token_logprob(logits, some), ref.token_logprob(logits, some), 1e-3, 1e-3)
    lb = logits.to(BF)
    ids2, _ = ops.sample(lb)
    assert ids2.tolist() == lb.float().argmax(-1).tolist()


@pytest.mark.parametrize("B,V", [(256, 128256), (1, 151936), (700, 2048), (3, 1000)])
def test_sampler_greedy_many_ctas(dev, B, V):
    torch.manual_seed(B)
    logits = torch.randn(B, V, device=dev) * 4
    logits[:, V // 3] = logits.max() + 1.0          # a tie between two columns: the lower index wins
    logits[:, V // 3 + 7] = logits[:, V // 3]
    ids, lp = ops.sample(logits)
    assert ids.tolist() == [V // 3] * B
    want = torch.log_softmax(logits.float(), dim=-1)[:, V // 3]
    close(lp, want, 1e-3, 1e-3)


@pytest.mark.parametrize("B,V,R", [(256, 128256, 8), (5, 32000, 2), (64, 151936, 4)])
def test_sampler_greedy_from_vocabulary_shards(dev, B, V, R):
    """The two greedy passes run per vocabulary shard (what R tensor-parallel ranks do) and merged give the
    token and log-probability of one pass over the whole row; the CPU restatement agrees."""
    torch.manual_seed(B + R)
    logits = torch.randn(B, V, device=dev) * 4
    logits[0, V - 1] = logits.max() + 2.0           # winner in the last shard
    logits[1 % B, 5] = logits.max() + 3.0           # tie across two shards: the lower token id wins
    logits[1 % B, V - 9] = logits[1 % B, 5]
    Vl = V // R
    parts = torch.stack([ops.greedy_partials(logits[:, r * Vl:(r + 1) * Vl], r * Vl) for r in range(R)])
    ids, lp = ops.greedy_merge(parts)
    want_ids = logits.argmax(-1)
    want_ids[1 % B] = 5
    assert ids.tolist() == want_ids.tolist()
    want_lp = torch.log_softmax(logits.float(), -1).gather(1, want_ids[:, None])[:, 0]
    close(lp, want_lp, 1e-3, 1e-3)
    lc = logits.cpu()
    parts_c = torch.stack([ops.greedy_partials(lc[:, r * Vl:(r + 1) * Vl], r * Vl) for r in range(R)])
    ids_c, lp_c = ops.greedy_merge(parts_c)
    assert ids_c.tolist() == want_ids.tolist()
    close(lp_c, want_lp.cpu(), 1e-3, 1e-3)


def test_sampler_topk_topp_support_and_distribution(dev):
    torch.manual_seed(7)
    V = 5000
    logits = (torch.randn(1, V, device=dev) * 2).repeat(4000, 1).contiguous()
    B = logits.shape[0]
    temp = torch.full((B,), 0.8, device=dev)
    top_p = torch.full((B,), 0.7, device=dev)
    top_k = torch.full((B,), 40, dtype=torch.int32, device=dev)
    seeds = torch.arange(B, device=dev, dtype=torch.int64) * 7919 + 13
    steps = torch.zeros(B, device=dev, dtype=torch.int64)
    ids, lp = ops.sample(logits, temp, top_p, top_k, seeds, steps)
    keep = ref.filtered_support(logits[0] / 0.8, 0.7, 40)
    assert keep[ids].all(), "sampled a token outside the top-k/top-p support"
    # empirical distribution close to the renormalised filtered softmax
    probs = torch.softmax(logits[0] / 0.8, -1) * keep
    probs = probs / probs.sum()
    counts = torch.bincount(ids, minlength=V).float() / B
    top = torch.argsort(probs, descending=True)[:5]
    assert (counts[top] - probs[top]).abs().max().item() < 0.04
    # determinism for a fixed seed, independence from batch position
    ids_b, _ = ops.sample(logits[:7], temp[:7], top_p[:7], top_k[:7], seeds[:7], steps[:7])
    assert ids_b.tolist() == ids[:7].tolist()


def test_penalties(dev):
    torch.manual_seed(8)
    B, V = 4, 1000
    logits = torch.randn(B, V, device=dev)
    l2 = logits.clone()
    pres = torch.tensor([0.5, 0, 0.1, 0], device=dev)
    freq = torch.tensor([0.2, 0, 0.0, 0.3], device=dev)
    rep = torch.tensor([1.2, 1.0, 1.0, 1.5], device=dev)
    cu = torch.tensor([0, 3, 3, 5, 6], dtype=torch.int32, device=dev)
    ids = torch.tensor([1, 5, 9, 2, 3, 999], dtype=torch.int32, device=dev)
    cnt = torch.tensor([1, 2, 3, 1, 4, 2], dtype=torch.int32, device=dev)
    mcu = torch.tensor([0, 0, 2, 2, 3], dtype=torch.int32, device=dev)
    mids = torch.tensor([7, 8, 0], dtype=torch.int32, device=dev)
    ops.apply_penalty_(logits, pres, freq, rep, cu, ids, cnt, mcu, mids)
    ref.apply_penalty_(l2, pres, freq, rep, cu, ids, cnt, mcu, mids)
    assert torch.equal(torch.isinf(logits), torch.isinf(l2))
    close(torch.nan_to_num(logits, neginf=0), torch.nan_to_num(l2, neginf=0), 1e-5, 1e-5)
