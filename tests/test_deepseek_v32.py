"""DeepSeek-V3.2 sparse attention on CPU: the selection path agrees with a brute-force restatement, prefill /
chunked prefill / decode give the same logits for the same positions, and short contexts take the dense path."""
import numpy as np
import torch

from lightllm_b200.common.infer_state import ModelInput
from lightllm_b200.models.registry import get_model
from lightllm_b200.parallel import dist as pdist

CFG = dict(model_type="deepseek_v32", hidden_size=64, intermediate_size=128, moe_intermediate_size=32,
           num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1,
           num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=32, kv_lora_rank=48,
           qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, vocab_size=200, max_position_embeddings=256,
           routed_scaling_factor=2.5, norm_topk_prob=True, rms_norm_eps=1e-6, index_n_heads=4, index_head_dim=16,
           index_topk=8)


def _model(**over):
    cfg = dict(CFG, **over)
    return get_model(cfg, pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                     max_total_token_num=512, max_req_num=4, max_seq_length=128, disable_cudagraph=True, random_seed=3)


def _prefill(m, req, ids, ready):
    n = len(ids)
    mi = ModelInput(batch_size=1, total_token_num=ready + n, max_kv_len=ready + n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32),
                    b_seq_len=torch.tensor([ready + n], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(n).clone(),
                    input_ids=ids, b_ready_cache_len=torch.tensor([ready], dtype=torch.int32), max_q_len=n,
                    return_all_logits=True)
    return m.forward(mi).logits.float()


def test_prefill_chunks_and_decode_agree_under_sparse_selection():
    m = _model()
    assert type(m).__name__ == "DeepseekV32LM" and m.index_k.shape == (3, 513, 16)
    ids = torch.randint(3, 200, (40,), generator=torch.Generator().manual_seed(0))
    whole = _prefill(m, m.req_manager.alloc(), ids, 0)
    r = m.req_manager.alloc()
    parts = [_prefill(m, r, ids[:10], 0), _prefill(m, r, ids[10:25], 10)]
    for t in range(25, 40):
        m.req_manager.req_to_next_token_ids[r] = int(ids[t])
        mi = ModelInput(batch_size=1, total_token_num=t + 1, max_kv_len=t + 1, is_prefill=False,
                        b_req_idx=torch.tensor([r], dtype=torch.int32), b_seq_len=torch.tensor([t + 1], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(1).clone())
        parts.append(m.forward(mi).logits.float())
    stepwise = torch.cat(parts)
    assert (whole - stepwise).abs().max().item() < 2e-4 * max(whole.abs().max().item(), 1.0)


def test_short_contexts_are_dense_and_long_ones_are_not():
    sparse, dense = _model(), _model(index_topk=1000)
    ids = torch.randint(3, 200, (30,), generator=torch.Generator().manual_seed(1))
    a = _prefill(sparse, sparse.req_manager.alloc(), ids[:8], 0)
    b = _prefill(dense, dense.req_manager.alloc(), ids[:8], 0)
    assert torch.equal(a, b)                                         # 8 tokens: everything is selected
    a = _prefill(sparse, sparse.req_manager.alloc(), ids, 0)
    b = _prefill(dense, dense.req_manager.alloc(), ids, 0)
    assert (a[:8] - b[:8]).abs().max().item() < 1e-5                 # the first 8 positions see at most 8 tokens
    assert (a[20:] - b[20:]).abs().max().item() > 1e-4               # later ones attend to a subset


def test_selection_against_brute_force():
    m = _model()
    seen = {}
    orig = m._sparse_attend

    def spy(qi, w, idx_layer, q_lat, q_pe, kv_layer, st):
        out = orig(qi, w, idx_layer, q_lat, q_pe, kv_layer, st)
        seen.setdefault("calls", []).append((qi.clone(), w.clone(), idx_layer.clone(), q_lat.clone(), q_pe.clone(),
                                             kv_layer.clone(), out.clone()))
        return out

    m._sparse_attend = spy
    ids = torch.randint(3, 200, (21,), generator=torch.Generator().manual_seed(2))
    req = m.req_manager.alloc()
    _prefill(m, req, ids, 0)
    qi, w, idx_layer, q_lat, q_pe, kv_layer, out = seen["calls"][0]
    slots = m.req_manager.req_to_token_indexs[req, :21].long()
    kvl, k = m.kv_lora, m.idx_topk
    for t in (0, 7, 8, 15, 20):
        scores = []
        for s in range(t + 1):
            kk = idx_layer[slots[s]].float()
            scores.append(sum(float(w[t, h]) * max(float(qi[t, h] @ kk), 0.0) for h in range(m.idx_heads)))
        order = sorted(range(t + 1), key=lambda s: -scores[s])[:k]
        rows = kv_layer[slots[order], 0].float()
        for h in range(q_lat.shape[1]):
            logit = (rows[:, :kvl] @ q_lat[t, h].float() + rows[:, kvl:] @ q_pe[t, h].float()) * m.sm_scale
            want = torch.softmax(logit, 0) @ rows[:, :kvl]
            assert (out[t, h].float() - want).abs().max().item() < 1e-4
