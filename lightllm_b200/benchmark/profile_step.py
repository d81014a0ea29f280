"""Small fixed workload for kernel profiling: a few transformer layers of a given architecture,
one prefill pass and a few decode steps, launched eagerly (no CUDA graph) so that every kernel
shows up as its own launch.

    python -m lightllm_b200.benchmark.profile_step --layers 4 --batch 256 --ctx 1024 --decode-steps 3
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--decode-steps", type=int, default=3)
    ap.add_argument("--prefill-tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    a = ap.parse_args()
    from lightllm_b200 import ops
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    dev = torch.device("cuda", 0)
    pdist.init_distributed(1, 0, device=dev)
    cfg = dict(model_type="llama", hidden_size=a.hidden, num_hidden_layers=a.layers, num_attention_heads=a.heads,
               num_key_value_heads=a.kv_heads, head_dim=128, intermediate_size=a.inter, vocab_size=a.vocab,
               rms_norm_eps=1e-5, rope_theta=5e5)
    B, L = a.batch, a.ctx
    m = get_model(cfg, max_total_token_num=B * (L + 16), max_req_num=B, max_seq_length=L + 32, disable_cudagraph=True)
    slots = m.mem_manager.alloc(B * (L + 8)).clone().view(B, L + 8)
    reqs = torch.arange(B, dtype=torch.int32)
    per = max(1, a.prefill_tokens // L)
    g = torch.Generator().manual_seed(0)
    for s in range(0, B, per):
        e = min(B, s + per)
        n = e - s
        mi = ModelInput(batch_size=n, total_token_num=n * L, max_kv_len=L, is_prefill=True, b_req_idx=reqs[s:e].clone(),
                        b_seq_len=torch.full((n,), L, dtype=torch.int32), mem_indexes=slots[s:e, :L].reshape(-1).clone(),
                        input_ids=torch.randint(0, a.vocab, (n * L,), generator=g),
                        b_ready_cache_len=torch.zeros(n, dtype=torch.int32), max_q_len=L)
        out = m.forward(mi)
        tok, _ = ops.sample(out.logits_any)
        ops.scatter_next_token_(m.req_manager.req_to_next_token_ids, tok, reqs[s:e].to(dev))
    torch.cuda.synchronize()
    for t in range(a.decode_steps):
        mi = ModelInput(batch_size=B, total_token_num=B * (L + t + 1), max_kv_len=L + t + 1, is_prefill=False,
                        b_req_idx=reqs.clone(), b_seq_len=torch.full((B,), L + t + 1, dtype=torch.int32),
                        mem_indexes=slots[:, L + t].clone())
        out = m.forward(mi)
        tok, _ = ops.sample(out.logits_any)
        ops.scatter_next_token_(m.req_manager.req_to_next_token_ids, tok, reqs.to(dev))
    torch.cuda.synchronize()
    print("profile_step done; gemm status", int(ops.gemm_status(dev).item()))


if __name__ == "__main__":
    main()
