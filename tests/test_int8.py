"""int8 w8a8: quantisers, CPU arithmetic, online quantisation of a model, and (on a GPU) the tcgen05 kind::i8 kernel
against the exact integer product."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import int8
from lightllm_b200.ops import reference as ref

BF = torch.bfloat16


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def test_int8_cpu_paths():
    torch.manual_seed(0)
    x = (torch.randn(50, 320) * 0.5).to(BF)
    w = torch.randn(192, 320) * 0.05
    iw = int8.Int8Weight.from_float(w)
    assert _rel(iw.dequant(), w) < 0.01
    want = x.float() @ w.t()
    assert _rel(ops.gemm(x, iw), want) < 0.03
    res = torch.randn(50, 192).to(BF)
    assert _rel(ops.gemm(x, iw, epi="residual", residual=res), want + res.float()) < 0.03
    wi = int8.Int8Weight.from_float(ref.interleave_gate_up(w[:96], w[96:]))
    want_g = torch.nn.functional.silu(x.float() @ w[:96].t()) * (x.float() @ w[96:].t())
    assert _rel(ops.gemm(x, wi, epi="gated_silu"), want_g) < 0.05


def test_online_int8_quantisation_of_a_model_cpu():
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    cfg = dict(model_type="llama", hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=1024)
    ids = torch.randint(3, 1000, (33,), generator=torch.Generator().manual_seed(0))

    def run(source=None, **kw):
        m = get_model(cfg, pstate=pdist.ParallelState(device=torch.device("cpu")), max_total_token_num=256,
                      max_req_num=2, max_seq_length=64, random_seed=1, weight_source=source, **kw)
        req, slots = m.req_manager.alloc(), m.mem_manager.alloc(len(ids))
        mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([len(ids)], dtype=torch.int32), mem_indexes=slots.clone(),
                        input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=len(ids),
                        return_all_logits=True)
        return m, m.forward(mi).logits.float()

    m16, want = run()
    m8, got = run(source=m16.weight_source, quant_type="w8a8")
    assert type(m8.layers[0].qkv_w).__name__ == "Int8Weight" and type(m8.layers[1].gate_up_w).__name__ == "Int8Weight"
    assert m8.param_bytes() < m16.param_bytes()
    assert ((got - want).norm() / want.norm()).item() < 0.1


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (1, 256, 512), (77, 512, 4096), (300, 4096, 512), (1000, 1536, 1536),
                                   (130, 264, 400)])
def test_gpu_int8_gemm_matches_the_integer_product(dev, M, N, K):
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = torch.randn(N, K, device=dev) * 0.05
    iw = int8.Int8Weight.from_float(w)
    xq, xs = int8.quant_act(x)
    xq_ref, xs_ref = int8.quant_act_reference(x)
    assert (xs - xs_ref).abs().max().item() <= 1e-6 * xs_ref.abs().max().item()
    assert (xq.int() - xq_ref.int()).abs().max().item() <= 1
    want = (xq.cpu().to(torch.int32) @ iw.q.cpu().to(torch.int32).t()).float().to(dev) * xs.unsqueeze(1) * \
        iw.scale.unsqueeze(0)
    got = int8.gemm_int8_quantized(xq, xs, iw)
    assert _rel(got, want) < 6e-3, "bf16 rounding of the output only"
    res = torch.randn(M, N, device=dev).to(BF)
    assert _rel(int8.gemm_int8_quantized(xq, xs, iw, "residual", residual=res), want + res.float()) < 6e-3
    assert int(ops.gemm_status(dev).item()) == 0
    assert _rel(ops.gemm(x, iw), x.float() @ w.t()) < 0.03


@pytest.mark.gpu
def test_gpu_int8_gated_epilogue(dev):
    torch.manual_seed(6)
    M, I, K = 200, 512, 1024
    x = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    g, u = torch.randn(I, K, device=dev) * 0.05, torch.randn(I, K, device=dev) * 0.05
    wi = int8.Int8Weight.from_float(ref.interleave_gate_up(g, u))
    want = torch.nn.functional.silu(x.float() @ g.t()) * (x.float() @ u.t())
    assert _rel(ops.gemm(x, wi, epi="gated_silu"), want) < 0.05


def test_awq_checkpoint_is_expanded_at_load(tmp_path):
    """4-bit AWQ packing round trip, and a Llama checkpoint stored in AWQ form gives the logits of its de-quantised
    weights."""
    import json
    import os

    from safetensors.torch import save_file

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models import quant
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    g = torch.Generator().manual_seed(0)
    vals = torch.randint(0, 16, (24, 64), generator=g, dtype=torch.int32)
    assert torch.equal(quant.awq_unpack(quant.awq_pack(vals)), vals)

    cfg = dict(model_type="llama", hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=300, torch_dtype="float32")
    ps = pdist.ParallelState(device=torch.device("cpu"))
    base = get_model(cfg, pstate=ps, data_type="float32", max_total_token_num=128, max_req_num=2, max_seq_length=64,
                     random_seed=5)
    tensors, dense = {}, {}
    group = 32
    for name in base.weight_source.names():
        w = base.weight_source.get(name).float()
        if name.endswith("proj.weight"):                       # quantise every Linear of the decoder layers
            N, K = w.shape
            wt = w.t().contiguous().view(K // group, group, N)
            lo, hi = wt.amin(1), wt.amax(1)
            scale = ((hi - lo) / 15).clamp_min(1e-8)
            zero = torch.round(-lo / scale).clamp(0, 15)
            q = torch.round(wt / scale.unsqueeze(1) + zero.unsqueeze(1)).clamp(0, 15)
            p = name[:-len("weight")]
            tensors[p + "qweight"] = quant.awq_pack(q.view(K, N).to(torch.int32))
            tensors[p + "qzeros"] = quant.awq_pack(zero.to(torch.int32))
            tensors[p + "scales"] = scale.to(torch.float16)
            dense[name] = quant.awq_dequant(tensors[p + "qweight"], tensors[p + "qzeros"], tensors[p + "scales"],
                                            torch.float32)
            assert (dense[name] - w).abs().max().item() < 0.6 * scale.max().item() + 1e-3
        else:
            tensors[name] = w.contiguous()
            dense[name] = w
    d = str(tmp_path / "awq")
    os.makedirs(d)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    json.dump({**cfg, "quantization_config": {"quant_method": "awq", "bits": 4, "group_size": group,
                                               "zero_point": True, "version": "gemm"}},
              open(os.path.join(d, "config.json"), "w"))

    class Dense:
        def has(self, n):
            return n in dense

        def names(self):
            return list(dense)

        def shape(self, n):
            return tuple(dense[n].shape)

        def get(self, n, dim=None, start=0, end=None):
            t = dense[n]
            return t if dim is None else t.narrow(dim, start, (t.shape[dim] if end is None else end) - start)

    ids = torch.randint(3, 290, (21,), generator=g)

    def logits(m):
        req, n = m.req_manager.alloc(), len(ids)
        mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                        b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True)
        return m.forward(mi).logits.float()

    from lightllm_b200.models.base import load_config

    awq = get_model(load_config(d), model_dir=d, pstate=ps, data_type="float32", max_total_token_num=128, max_req_num=2,
                    max_seq_length=64)
    want = get_model(cfg, pstate=ps, data_type="float32", max_total_token_num=128, max_req_num=2, max_seq_length=64,
                     weight_source=Dense())
    assert (logits(awq) - logits(want)).abs().max().item() < 1e-4
