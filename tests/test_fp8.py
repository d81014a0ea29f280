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


DSV3_FP8 = dict(model_type="deepseek_v3", hidden_size=512, intermediate_size=1024, moe_intermediate_size=256,
                num_hidden_layers=3, num_attention_heads=4, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
                qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                first_k_dense_replace=1, moe_layer_freq=1, n_group=2, topk_group=1, vocab_size=1024,
                rms_norm_eps=1e-6, rope_theta=10000.0, routed_scaling_factor=2.5, norm_topk_prob=True, eos_token_id=2,
                quantization_config=dict(quant_method="fp8", weight_block_size=[128, 128]))


def _prefill_logits(device, source=None, **kw):
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    m = get_model(DSV3_FP8, pstate=pdist.ParallelState(device=device), max_total_token_num=512, max_req_num=4,
                  max_seq_length=128, random_seed=3, disable_cudagraph=True, weight_source=source, **kw)
    ids = torch.randint(3, 1000, (40,), generator=torch.Generator().manual_seed(0))
    req = m.req_manager.alloc()
    slots = m.mem_manager.alloc(len(ids))
    mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32),
                    b_seq_len=torch.tensor([len(ids)], dtype=torch.int32), mem_indexes=slots.clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=len(ids), return_all_logits=True)
    return m, m.forward(mi).logits.float().cpu()


def test_deepseek_fp8_checkpoint_runs_on_fp8_weights_cpu():
    """An fp8 block-quantised checkpoint keeps its experts, dense FFN, q_b and o_proj in e4m3 (half the bytes) and
    stays close to the path that expands everything to bf16 (the difference is the activation quantisation)."""
    m8, a = _prefill_logits(torch.device("cpu"))
    m16, b = _prefill_logits(torch.device("cpu"), source=m8.weight_source, dequant_fp8=True)
    assert type(m8.layers[1].w13).__name__ == "Fp8Experts" and type(m8.layers[0].gate_up_w).__name__ == "Fp8Weight"
    assert type(m8.layers[0].o_w).__name__ == "Fp8Weight" and type(m8.layers[0].q_b_w).__name__ == "Fp8Weight"
    assert isinstance(m16.layers[1].w13, torch.Tensor)
    assert m8.param_bytes() < 0.7 * m16.param_bytes()
    assert ((a - b).norm() / b.norm()).item() < 0.25


@pytest.mark.gpu
def test_deepseek_fp8_gpu_matches_cpu(dev):
    mc, c = _prefill_logits(torch.device("cpu"))
    mg, g = _prefill_logits(dev, source=mc.weight_source)
    assert type(mg.layers[1].w13).__name__ == "Fp8Experts"
    # same quantised operands on both sides, but the device quantiser multiplies by the reciprocal scale (values on a
    # rounding boundary move one e4m3 step) and a router near-tie can flip an expert for a token: most tokens agree
    # closely, single tokens may not
    per_token = (g - c).norm(dim=1) / c.norm(dim=1)
    assert per_token.median().item() < 0.1 and ((g - c).norm() / c.norm()).item() < 0.35
    assert int(ops.gemm_status(dev).item()) == 0


@pytest.mark.parametrize("family", ["llama", "qwen3_moe"])
def test_online_fp8_quantisation_of_bf16_checkpoints_cpu(family, tmp_path):
    """`--quant_type fp8w8a8*` on an unquantised model: the big matrices become block-scaled e4m3 at load and the
    logits stay close to the unquantised network; a `--quant_cfg` YAML can keep single layers in bf16."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.common.quantization import QuantConfig, canonical
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    cfgs = {
        "llama": dict(model_type="llama", hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=1024),
        "qwen3_moe": dict(model_type="qwen3_moe", hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
                          num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                          num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                          mlp_only_layers=[], vocab_size=1024),
    }
    ids = torch.randint(3, 1000, (33,), generator=torch.Generator().manual_seed(0))

    def run(source=None, **kw):
        m = get_model(cfgs[family], pstate=pdist.ParallelState(device=torch.device("cpu")), max_total_token_num=256,
                      max_req_num=2, max_seq_length=64, random_seed=1, weight_source=source, **kw)
        req, slots = m.req_manager.alloc(), m.mem_manager.alloc(len(ids))
        mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([len(ids)], dtype=torch.int32), mem_indexes=slots.clone(),
                        input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=len(ids),
                        return_all_logits=True)
        return m, m.forward(mi).logits.float()

    m16, want = run()
    m8, got = run(source=m16.weight_source, quant_type="fp8w8a8")
    assert type(m8.layers[0].qkv_w).__name__ == "Fp8Weight" and type(m8.layers[1].o_w).__name__ == "Fp8Weight"
    if family == "qwen3_moe":
        assert type(m8.layers[0].w13).__name__ == "Fp8Experts"
    else:
        assert m8.layers[0].gate_up_w.ws_rows == 32
    assert ((got - want).norm() / want.norm()).item() < 0.2
    y = tmp_path / "q.yaml"
    y.write_text("quant_type: fp8w8a8-b128\nmix_bits:\n  - layer_nums: [1]\n    quant_type: none\n")
    mm, _ = run(source=m16.weight_source, quant_cfg=str(y))
    assert type(mm.layers[0].qkv_w).__name__ == "Fp8Weight" and isinstance(mm.layers[1].qkv_w, torch.Tensor)
    assert canonical("fp8w8a8-b128-deepgemm") == "fp8w8a8-b128"
    with pytest.raises(NotImplementedError):
        canonical("awq_marlin")
    assert QuantConfig({"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}).default == \
        "fp8w8a8-b128"
