"""Gated DeltaNet building blocks: the chunked and single-step forms against the token-by-token definition, the
causal convolution with carried state."""
import torch

from lightllm_b200.ops import linear_attn as la


def _inputs(T, H=3, dk=16, dv=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(T, H, dk, generator=g), torch.randn(T, H, dk, generator=g)
    v = torch.randn(T, H, dv, generator=g)
    decay = -torch.rand(T, H, generator=g) * 0.5
    beta = torch.rand(T, H, generator=g)
    return q, k, v, decay, beta


def test_chunked_and_step_forms_match_the_recurrence():
    q, k, v, g, beta = _inputs(150)
    want, S_want = la.gated_delta_naive(q, k, v, g, beta)
    got, S_got = la.gated_delta_chunked(q, k, v, g, beta, chunk=64)
    assert (got - want).abs().max().item() < 1e-4 and (S_got - S_want).abs().max().item() < 1e-4
    # a prompt processed in two pieces (chunked prefill) carries the state over
    o1, S1 = la.gated_delta_chunked(q[:70], k[:70], v[:70], g[:70], beta[:70], chunk=32)
    o2, S2 = la.gated_delta_chunked(q[70:], k[70:], v[70:], g[70:], beta[70:], S0=S1, chunk=32)
    assert (torch.cat([o1, o2]) - want).abs().max().item() < 1e-4 and (S2 - S_want).abs().max().item() < 1e-4
    # decode steps of a batch of two requests continue from their own states
    S = torch.stack([S1, S_want])
    o, Sn = la.gated_delta_step(torch.stack([q[70], q[0]]), torch.stack([k[70], k[0]]), torch.stack([v[70], v[0]]),
                                torch.stack([g[70], g[0]]), torch.stack([beta[70], beta[0]]), S)
    assert (o[0] - want[70]).abs().max().item() < 1e-4
    ref1, _ = la.gated_delta_naive(q[:1], k[:1], v[:1], g[:1], beta[:1], S0=S_want)
    assert (o[1] - ref1[0]).abs().max().item() < 1e-4


def test_causal_conv_state_carry():
    torch.manual_seed(1)
    C, K, T = 10, 4, 23
    x, w = torch.randn(T, C), torch.randn(C, K)
    full, st = la.causal_conv_prefill(x, torch.zeros(C, K - 1), w)
    want = torch.nn.functional.silu(torch.nn.functional.conv1d(
        torch.nn.functional.pad(x.t().unsqueeze(0), (K - 1, 0)), w.unsqueeze(1), groups=C))[0].t()
    assert (full - want).abs().max().item() < 1e-5
    a, sa = la.causal_conv_prefill(x[:9], torch.zeros(C, K - 1), w)
    b, sb = la.causal_conv_prefill(x[9:22], sa, w)
    step, sc = la.causal_conv_step(x[22:23], sb.unsqueeze(0), w)
    assert (torch.cat([a, b, step]) - want).abs().max().item() < 1e-5
    assert (sc[0] - st).abs().max().item() < 1e-6


def test_qwen3_next_serves_batches_through_the_engine():
    """Continuous batching over a hybrid model: several requests with different prompt lengths decode together and
    give the same tokens as each request alone (per-request convolution / matrix state, no prefix sharing)."""
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="qwen3_next", hidden_size=64, intermediate_size=128, moe_intermediate_size=32,
               shared_expert_intermediate_size=32, num_experts=4, num_experts_per_tok=2, num_hidden_layers=4,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=300, linear_num_value_heads=4,
               linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
               full_attention_interval=4, partial_rotary_factor=0.25, norm_topk_prob=True, eos_token_id=2,
               rms_norm_eps=1e-6)
    llm = LLM(config=cfg, max_total_token_num=2048, running_max_req_size=4, max_req_total_len=256,
              batch_max_tokens=64, data_type="float32")
    assert llm.backend.radix_cache is None
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 290, (n,), generator=g).tolist() for n in (9, 70, 33)]   # 70 > batch_max_tokens: chunked
    together = llm.generate(prompts, {"max_new_tokens": 6, "ignore_eos": True})
    for p, out in zip(prompts, together):
        alone = llm.generate([p], {"max_new_tokens": 6, "ignore_eos": True})[0]
        assert alone["token_ids"] == out["token_ids"]
