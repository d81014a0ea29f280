"""MLA kernels (rope + latent norm + scatter, per-head batched GEMM, absorbed attention) against fp32
PyTorch restatements."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import mla
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
KVL, ROPE, NOPE = 512, 64, 128


def test_mla_rope_kv_scatter(dev):
    torch.manual_seed(0)
    T, hq, slots = 37, 16, 100
    q3 = torch.randn(T, hq, NOPE + ROPE, device=dev, dtype=BF)
    big = torch.randn(T, 1536 + KVL + ROPE, device=dev, dtype=BF)
    kv_a = big[:, 1536:]  # strided view, as in the fused q_a / kv_a GEMM output
    pool = torch.zeros(slots, 1, KVL + ROPE, device=dev, dtype=BF)
    w = (torch.randn(KVL, device=dev) * 0.1 + 1).to(BF)
    cos, sin = ref.build_rope_cache(256, ROPE, 1e4, None, device=dev)
    pos = torch.randint(0, 256, (T,), device=dev, dtype=torch.int32)
    slot = torch.randperm(slots, device=dev)[:T].to(torch.int32)
    q_ref, pool_ref = q3.clone(), pool.clone()
    ref.mla_rope_kv_scatter_(q_ref, kv_a, pool_ref, w, cos, sin, pos, slot, NOPE, ROPE, KVL, 1e-6)
    ops.mla_rope_kv_scatter_(q3, kv_a, pool, w, cos, sin, pos, slot, NOPE, ROPE, KVL, 1e-6)
    assert (q3.float() - q_ref.float()).abs().max().item() < 5e-2
    assert (pool.float() - pool_ref.float()).abs().max().item() < 5e-2


@pytest.mark.parametrize("T,h,N,K", [(5, 16, 512, 128), (300, 16, 512, 128), (64, 128, 128, 512), (257, 4, 128, 512)])
def test_gemm_batched(dev, T, h, N, K):
    torch.manual_seed(1)
    wide = (torch.randn(T, h, K + 64, device=dev) * 0.5).to(BF)
    a = wide[:, :, :K]  # per-head slice of a wider row, like q_nope inside q
    w = (torch.randn(h, N, K, device=dev) * 0.1).to(BF)
    got = mla.gemm_batched(a, w)
    want = torch.einsum("thk,hnk->thn", a.float(), w.float())
    err = (got.float() - want).abs().max().item()
    assert err < 1e-2 * want.abs().max().item() + 1e-2, err
    assert int(ops.gemm_status(dev).item()) == 0


def _case(dev, ready, new, hq, seed):
    g = torch.Generator().manual_seed(seed)
    lens = [r + n for r, n in zip(ready, new)]
    total = sum(lens)
    pool = (torch.randn(total + 9, 1, KVL + ROPE, generator=g) * 0.3).to(dev, BF)
    perm = torch.randperm(total + 8, generator=g)[:total].to(torch.int32)
    r2t = torch.zeros(len(lens) + 1, max(lens) + 2, dtype=torch.int32)
    off = 0
    for i, L in enumerate(lens):
        r2t[i, :L] = perm[off:off + L]
        off += L
    T = sum(new)
    q_lat = (torch.randn(T, hq, KVL, generator=g) * 0.3).to(dev, BF)
    q = (torch.randn(T, hq, NOPE + ROPE, generator=g) * 0.3).to(dev, BF)
    q_pe = q[:, :, NOPE:]
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev)
    b_of = torch.repeat_interleave(torch.arange(len(new)), torch.tensor(new)).to(torch.int32).to(dev)
    return (q_lat, q_pe, pool, r2t.to(dev), torch.arange(len(lens), dtype=torch.int32, device=dev),
            torch.tensor(lens, dtype=torch.int32, device=dev), cu, torch.tensor(ready, dtype=torch.int32, device=dev), b_of)


@pytest.mark.parametrize("hq", [16, 128, 8])
def test_mla_attention_decode_and_prefill(dev, hq):
    scale = 0.07
    # decode: one new token per request on top of a cached context
    ready = [0, 63, 64, 300, 1000]
    q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, b_of = _case(dev, ready, [1] * 5, hq, 0)
    got = mla.mla_attention(q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, KVL, scale, False)
    want = mla.ref_mla_attention(q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, KVL, scale)
    assert (got.float() - want.float()).abs().max().item() < 2e-2
    # prefill: causal over cached prefix + new tokens
    q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, b_of = _case(dev, [0, 40, 0], [70, 33, 1], hq, 1)
    got = mla.mla_attention(q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, KVL, scale, True, 70, 0, batch_of=b_of)
    want = mla.ref_mla_attention(q_lat, q_pe, pool, r2t, b_req, b_len, cu, rdy, KVL, scale)
    assert (got.float() - want.float()).abs().max().item() < 2e-2


def test_deepseek_tiny_model_gpu_matches_cpu(dev):
    """Whole DeepSeek-V3-style layer stack (MLA + dense + MoE with shared expert) on the kernels vs the fp32
    restatement path on CPU, same random weights."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    cfg = dict(model_type="deepseek_v3", hidden_size=512, num_hidden_layers=3, num_attention_heads=16, q_lora_rank=256,
               kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, intermediate_size=1024,
               moe_intermediate_size=256, n_routed_experts=16, n_shared_experts=1, num_experts_per_tok=4, n_group=4,
               topk_group=2, first_k_dense_replace=1, routed_scaling_factor=2.5, scoring_func="sigmoid",
               topk_method="noaux_tc", norm_topk_prob=True, vocab_size=2048, rms_norm_eps=1e-6, rope_theta=1e4,
               eos_token_id=2)
    ids = torch.randint(3, 2048, (150,), generator=torch.Generator().manual_seed(0))
    outs = {}
    source = None  # both models read the same CPU-generated tensors (a CUDA generator draws other numbers)
    for name, device in (("cpu", torch.device("cpu")), ("gpu", dev)):
        ps = pdist.ParallelState(device=device)
        m = get_model(cfg, pstate=ps, data_type="bfloat16" if name == "gpu" else "float32", max_total_token_num=1024,
                      max_req_num=4, max_seq_length=256, disable_cudagraph=True, random_seed=0, weight_source=source)
        source = m.weight_source
        req = m.req_manager.alloc()
        slots = m.mem_manager.alloc(len(ids))
        mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([len(ids)], dtype=torch.int32), mem_indexes=slots.clone(),
                        input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=len(ids))
        outs[name] = m.forward(mi).logits.float().cpu()
    scale = outs["cpu"].abs().max().item()
    err = (outs["cpu"] - outs["gpu"]).abs().max().item()
    assert err < 0.08 * scale + 0.05, (err, scale)


def test_deepseek_v32_sparse_attention_gpu_matches_cpu(dev):
    """DeepSeek-V3.2: contexts beyond `index_topk` select their keys with the indexer and attend through the MLA
    kernel over per-token slot lists (prompt pass and a decode step); the fp32 CPU restatement takes the same route
    on torch ops.  A near-tie in the selection can flip one key under bf16 rounding: the mean error is bounded
    tightly, the worst element loosely."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    cfg = dict(model_type="deepseek_v32", hidden_size=512, num_hidden_layers=3, num_attention_heads=16, q_lora_rank=256,
               kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, intermediate_size=1024,
               moe_intermediate_size=256, n_routed_experts=16, n_shared_experts=1, num_experts_per_tok=4, n_group=4,
               topk_group=2, first_k_dense_replace=1, routed_scaling_factor=2.5, scoring_func="sigmoid",
               topk_method="noaux_tc", norm_topk_prob=True, vocab_size=2048, rms_norm_eps=1e-6, rope_theta=1e4,
               eos_token_id=2, index_n_heads=16, index_head_dim=64, index_topk=64, max_position_embeddings=512)
    ids = torch.randint(3, 2048, (150,), generator=torch.Generator().manual_seed(0))
    outs = {}
    source = None
    for name, device in (("cpu", torch.device("cpu")), ("gpu", dev)):
        ps = pdist.ParallelState(device=device)
        m = get_model(cfg, pstate=ps, data_type="bfloat16" if name == "gpu" else "float32", max_total_token_num=1024,
                      max_req_num=4, max_seq_length=256, disable_cudagraph=True, random_seed=0, weight_source=source)
        source = m.weight_source
        calls = []
        orig = m._sparse_attend
        m._sparse_attend = lambda *a, _o=orig, _c=calls: (_c.append(1), _o(*a))[1]
        req = m.req_manager.alloc()
        slots = m.mem_manager.alloc(len(ids))
        mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([len(ids)], dtype=torch.int32), mem_indexes=slots.clone(),
                        input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=len(ids),
                        return_all_logits=True)
        pre = m.forward(mi).logits.float().cpu()
        m.req_manager.req_to_next_token_ids[req] = 17
        mi = ModelInput(batch_size=1, total_token_num=151, max_kv_len=151, is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([151], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(1).clone())
        dec = m.forward(mi).logits.float().cpu()
        outs[name] = torch.cat([pre, dec])
        assert len(calls) == 2 * 3                       # the selection route ran in every layer of both passes
    scale = outs["cpu"].abs().max().item()
    d = (outs["cpu"] - outs["gpu"]).abs()
    assert d.mean().item() < 0.02 * scale, (d.mean().item(), scale)
    assert d.max().item() < 0.5 * scale, (d.max().item(), scale)
    assert d[:64].max().item() < 0.08 * scale + 0.05     # the first index_topk positions select everything
