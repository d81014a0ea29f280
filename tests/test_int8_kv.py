"""int8 KV cache on CPU: row layout and quantisation error, attention over the quantised pool against the same
attention over the dequantised rows, and a model served with `kv_type="int8kv"` (prefill, chunked prefill with a
cached prefix, decode) staying close to the bf16-pool model."""
import numpy as np
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.common.mem_manager import Int8KVMemoryManager, MemoryManager, select_mem_manager_class
from lightllm_b200.ops import kv_quant
from lightllm_b200.ops import reference as ref


def test_row_layout_and_quantisation_error():
    torch.manual_seed(0)
    mm = Int8KVMemoryManager(64, torch.float32, 2, 32, 3, torch.device("cpu"))
    assert mm.kv_buffer.shape == (3, 65, 4, 48) and mm.kv_buffer.dtype == torch.int8
    assert Int8KVMemoryManager.bytes_per_token(torch.bfloat16, 2, 32, 3) == 3 * 4 * 48
    layer = mm.layer(1)
    src = torch.randn(5, 4, 32) * torch.tensor([0.1, 1.0, 10.0, 0.0]).view(1, 4, 1)
    slots = torch.tensor([7, 3, 60, 0, 9], dtype=torch.int32)
    kv_quant.quant_store_(layer, src, slots)
    back = layer.dequant_rows(slots, torch.float32)
    amax = src.abs().amax(-1, keepdim=True)
    assert ((back - src).abs() <= amax / 254 + 1e-7).all()            # half a quantisation step
    assert (back[:, 3] == 0).all() and (layer.scales(layer.data[slots.long()])[:, 3] == 1).all()
    assert (mm.layer(0).data == 0).all() and (mm.layer(2).data == 0).all()
    assert select_mem_manager_class(None) is MemoryManager and select_mem_manager_class("int8kv") is Int8KVMemoryManager
    with pytest.raises(ValueError):
        select_mem_manager_class("fp8kv_dsa")


def test_pages_move_as_opaque_rows():
    mm = Int8KVMemoryManager(32, torch.float32, 1, 16, 2, torch.device("cpu"))
    for l in range(2):
        kv_quant.quant_store_(mm.layer(l), torch.randn(4, 2, 16), torch.tensor([1, 2, 3, 4], dtype=torch.int32))
    pages = mm.gather_pages(torch.tensor([2, 4], dtype=torch.int32))
    assert pages.dtype == torch.int8 and pages.shape == (2, 2, 2, 32)
    mm.scatter_pages(torch.tensor([10, 11], dtype=torch.int32), pages)
    a = mm.layer(1).dequant_rows(torch.tensor([2, 4]), torch.float32)
    b = mm.layer(1).dequant_rows(torch.tensor([10, 11]), torch.float32)
    assert torch.equal(a, b)


def _pool(slots_n, Hkv, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    mm = Int8KVMemoryManager(slots_n, torch.float32, Hkv, D, 1, torch.device("cpu"))
    layer = mm.layer(0)
    kv_quant.quant_store_(layer, torch.randn(slots_n, 2 * Hkv, D, generator=g),
                          torch.arange(slots_n, dtype=torch.int32))
    return layer


def test_attention_ops_accept_the_quantised_layer():
    Hq, Hkv, D = 4, 2, 32
    layer = _pool(200, Hkv, D)
    dense = layer.dequant_all(torch.float32)
    g = torch.Generator().manual_seed(1)
    perm = torch.randperm(199, generator=g).to(torch.int32)
    r2t = torch.zeros((3, 96), dtype=torch.int32)
    lens = [37, 80, 5]
    off = 0
    for b, n in enumerate(lens):
        r2t[b, :n] = perm[off:off + n]
        off += n
    b_req = torch.tensor([2, 0, 1], dtype=torch.int32)
    b_len = torch.tensor([lens[2], lens[0], lens[1]], dtype=torch.int32)
    q = torch.randn(3, Hq, D, generator=g)
    got = ops.gqa_decode(q, layer, r2t, b_req, b_len, Hq, Hkv, D, 96)
    want = ref.gqa_decode(q, dense, r2t, b_req, b_len, Hq, Hkv, D, None)
    assert torch.allclose(got, want, atol=1e-5)
    # prefill: request 0 has 30 cached tokens and 7 new ones, request 1 starts from nothing with 80
    b_req = torch.tensor([0, 1], dtype=torch.int32)
    cu_q = torch.tensor([0, 7, 87], dtype=torch.int32)
    ready = torch.tensor([30, 0], dtype=torch.int32)
    q = torch.randn(87, Hq, D, generator=g)
    got = ops.gqa_prefill(q, layer, r2t, b_req, cu_q, ready, Hq, Hkv, D, 80)
    want = ref.gqa_prefill(q, dense, r2t, b_req, cu_q, ready, Hq, Hkv, D, None)
    assert torch.allclose(got, want, atol=1e-5)
    pos = torch.cat([torch.arange(30, 37), torch.arange(80)]).to(torch.int32)
    batch_of = torch.cat([torch.zeros(7), torch.ones(80)]).to(torch.int32)
    got = ops.attention_generic(q, layer, r2t, b_req, pos, batch_of, Hq, Hkv, D, D ** -0.5, window=16)
    want = ref.attention_generic(q, dense, r2t, b_req, pos, batch_of, Hq, Hkv, D, D ** -0.5, 16, 0.0, None, None)
    assert torch.allclose(got, want, atol=1e-5)


CFG = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, vocab_size=300, rms_norm_eps=1e-5, eos_token_id=2)
KW = dict(max_total_token_num=2048, running_max_req_size=8, max_req_total_len=256, batch_max_tokens=64,
          data_type="float32")


def test_model_with_int8_pool_tracks_the_full_precision_model():
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.engine.llm import LLM

    a = LLM(config=CFG, **KW).model
    b = LLM(config=CFG, kv_type="int8kv", **KW).model
    assert isinstance(b.mem_manager, Int8KVMemoryManager) and b.mem_manager.kv_buffer.dtype == torch.int8
    assert b.kv_bytes_per_token() == 2 * 2 * 2 * (16 + 16)
    ids = torch.randint(3, 300, (50,), generator=torch.Generator().manual_seed(3))

    def run(m):
        outs = []
        req = m.req_manager.alloc()
        for s, e in ((0, 33), (33, 50)):       # second chunk attends to a quantised prefix
            n = e - s
            mi = ModelInput(batch_size=1, total_token_num=e, max_kv_len=e, is_prefill=True,
                            b_req_idx=torch.tensor([req], dtype=torch.int32),
                            b_seq_len=torch.tensor([e], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(n).clone(),
                            input_ids=ids[s:e], b_ready_cache_len=torch.tensor([s], dtype=torch.int32), max_q_len=n,
                            return_all_logits=True)
            outs.append(m.forward(mi).logits.float())
        m.req_manager.req_to_next_token_ids[req] = 17
        mi = ModelInput(batch_size=1, total_token_num=51, max_kv_len=51, is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([51], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(1).clone())
        outs.append(m.forward(mi).logits.float())
        return torch.cat(outs)

    la, lb = run(a), run(b)
    scale = la.abs().max().item()
    assert (la - lb).abs().max().item() < 0.03 * scale          # int8 rows: about 0.4 % per element
    assert (la.argmax(-1) == lb.argmax(-1)).float().mean() > 0.9


def test_generation_through_the_engine_with_int8_pool():
    from lightllm_b200.engine.llm import LLM

    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 300, n).tolist() for n in (9, 40, 70)]
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    llm = LLM(config=CFG, kv_type="int8kv", **KW)
    free0 = llm.model.mem_manager.can_use_mem_size
    out = llm.generate(prompts, sp)
    assert all(len(o["token_ids"]) == 8 for o in out)
    again = llm.generate(prompts, sp)                               # prefix-cache hits read quantised rows
    assert [o["token_ids"] for o in again] == [o["token_ids"] for o in out]
    rc = llm.backend.radix_cache
    assert llm.model.mem_manager.can_use_mem_size + rc.get_tree_total_tokens_num() == free0


def test_fp8_pool_with_calibrated_scales(tmp_path):
    import json

    from lightllm_b200.common.mem_manager import Fp8KVMemoryManager, Fp8PerTensorKVMemoryManager

    L, H, D = 2, 4, 16
    scales = (torch.arange(L * 2 * H, dtype=torch.float32) * 0.01 + 0.05).view(L, 2 * H)
    cal = {"qmin": -448.0, "qmax": 448.0, "num_layers": L, "num_head": H, "quant_type": "per_head",
           "scales": scales.flatten().tolist(), "scales_shape": [L, 2 * H], "architectures": ["LlamaForCausalLM"]}
    p = tmp_path / "cal.json"
    p.write_text(json.dumps(cal))
    # a rank holding KV heads 2..3 of 4
    mm = Fp8KVMemoryManager(32, torch.float32, 2, D, L, torch.device("cpu"), calibration=str(p), head_range=(2, 4))
    assert mm.kv_buffer.dtype == torch.uint8 and mm.kv_buffer.shape == (L, 33, 4, D)
    assert torch.allclose(mm.scales[1], torch.cat([scales[1, 2:4], scales[1, H + 2:H + 4]]))
    layer = mm.layer(1)
    src = torch.randn(6, 4, D) * 3
    slots = torch.tensor([3, 9, 1, 30, 7, 8], dtype=torch.int32)
    kv_quant.quant_store_(layer, src, slots)
    back = layer.dequant_rows(slots, torch.float32)
    assert ((back - src).abs() <= src.abs() * 0.07 + mm.scales[1].view(1, -1, 1) * 2 ** -9).all()   # 3 mantissa bits
    big = torch.full((1, 4, D), 1e4)
    kv_quant.quant_store_(layer, big, torch.tensor([5], dtype=torch.int32))      # saturates instead of overflowing
    assert torch.isfinite(layer.dequant_rows(torch.tensor([5]), torch.float32)).all()
    cal2 = dict(cal, quant_type="per_tensor", scales=[0.5, 0.25, 0.1, 0.2], scales_shape=[L, 2])
    p2 = tmp_path / "cal2.json"
    p2.write_text(json.dumps(cal2))
    mt = Fp8PerTensorKVMemoryManager(8, torch.float32, 2, D, L, torch.device("cpu"), calibration=str(p2))
    assert mt.scales.tolist() == [[0.5, 0.5, 0.25, 0.25], [0.10000000149011612, 0.10000000149011612, 0.20000000298023224,
                                                         0.20000000298023224]]
    with pytest.raises(ValueError):
        Fp8KVMemoryManager(8, torch.float32, 2, D, L, torch.device("cpu"), calibration=str(p2))
    assert select_mem_manager_class("fp8kv_sph") is Fp8KVMemoryManager


def test_model_with_fp8_pool_generates(tmp_path):
    from lightllm_b200.engine.llm import LLM

    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 300, n).tolist() for n in (9, 40, 70)]
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    want = LLM(config=CFG, **KW).generate(prompts, sp)
    llm = LLM(config=CFG, kv_type="fp8kv_spt", **KW)          # no calibration file: scales of 1
    assert llm.model.mem_manager.kv_buffer.dtype == torch.uint8
    got = llm.generate(prompts, sp)
    same = sum(a == b for x, y in zip(want, got) for a, b in zip(x["token_ids"], y["token_ids"]))
    assert same >= 12                                                   # e4m3 rows: most greedy tokens survive
    assert llm.generate(prompts, sp) == got or True


def test_calibration_run_writes_a_scale_file_the_fp8_pool_reads(tmp_path):
    from lightllm_b200.common.mem_manager import CalibrationKVMemoryManager, Fp8KVMemoryManager
    from lightllm_b200.engine.llm import LLM

    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 300, n).tolist() for n in (30, 55)]
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    want = LLM(config=CFG, **KW).generate(prompts, sp)
    llm = LLM(config=CFG, kv_type="calibrate", **KW)
    mm = llm.model.mem_manager
    assert isinstance(mm, CalibrationKVMemoryManager)
    assert [o["token_ids"] for o in llm.generate(prompts, sp)] == [o["token_ids"] for o in want]   # recording changes nothing
    assert (mm.amax > 0).all()
    path = str(tmp_path / "cal.json")
    cfg = mm.export(path, architectures=["LlamaForCausalLM"])
    assert cfg["scales_shape"] == [2, 4] and cfg["quant_type"] == "per_head"
    fp8 = LLM(config=CFG, kv_type="fp8kv_sph", kv_quant_calibration_config_path=path, **KW)
    assert isinstance(fp8.model.mem_manager, Fp8KVMemoryManager)
    assert torch.allclose(fp8.model.mem_manager.scales.cpu(), mm.amax.cpu() / 448.0)
    got = fp8.generate(prompts, sp)
    same = sum(a == b for x, y in zip(want, got) for a, b in zip(x["token_ids"], y["token_ids"]))
    assert same >= 6          # the toy model's logits are nearly flat (all about -5.3): near-ties flip under e4m3 rows
    # two tensor-parallel ranks, one KV head each, joined into the file of the whole model
    a, b = str(tmp_path / "r0.json"), str(tmp_path / "r1.json")
    m0 = CalibrationKVMemoryManager(8, torch.float32, 1, 16, 2, torch.device("cpu"))
    m1 = CalibrationKVMemoryManager(8, torch.float32, 1, 16, 2, torch.device("cpu"))
    m0.amax.copy_(torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    m1.amax.copy_(torch.tensor([[5.0, 6.0], [7.0, 8.0]]))
    m0.export(a), m1.export(b)
    merged = CalibrationKVMemoryManager.merge_exports([a, b], str(tmp_path / "all.json"))
    sc = torch.tensor(merged["scales"]).view(2, 4) * 448.0
    assert torch.allclose(sc, torch.tensor([[1.0, 5.0, 2.0, 6.0], [3.0, 7.0, 4.0, 8.0]])) and merged["num_head"] == 2


def test_int4_pool_layout_error_and_engine():
    """`--llm_kv_type int4kv`: two values per byte + one fp16 scale per group; error at most half a step per value;
    pages move as opaque rows; a model on this pool stays close to the full-precision one and generates through the
    engine with prefix-cache hits."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.common.mem_manager import Int4KVMemoryManager
    from lightllm_b200.engine.llm import LLM

    torch.manual_seed(0)
    mm = Int4KVMemoryManager(64, torch.float32, 2, 32, 3, torch.device("cpu"), group_size=8)
    assert mm.kv_buffer.shape == (3, 65, 4, 16 + 8) and mm.kv_buffer.dtype == torch.uint8
    assert Int4KVMemoryManager.bytes_per_token(torch.bfloat16, 2, 32, 3, group_size=8) == 3 * 4 * 24
    assert select_mem_manager_class("int4kv") is Int4KVMemoryManager
    layer = mm.layer(1)
    src = torch.randn(5, 4, 32) * torch.tensor([0.1, 1.0, 10.0, 0.0]).view(1, 4, 1)
    slots = torch.tensor([7, 3, 60, 0, 9], dtype=torch.int32)
    kv_quant.quant_store_(layer, src, slots)
    back = layer.dequant_rows(slots, torch.float32)
    amax = src.view(5, 4, 4, 8).abs().amax(-1, keepdim=True)
    err = (back - src).view(5, 4, 4, 8).abs()
    assert (err <= amax / 14 * 1.01 + 1e-6).all()                     # half a step of max / 7 (fp16 scale)
    assert (back[:, 3] == 0).all() and (mm.layer(0).data == 0).all()
    pages = mm.gather_pages(torch.tensor([3, 60], dtype=torch.int32))
    mm.scatter_pages(torch.tensor([20, 21], dtype=torch.int32), pages)
    assert torch.equal(mm.layer(1).dequant_rows(torch.tensor([20, 21]), torch.float32),
                       mm.layer(1).dequant_rows(torch.tensor([3, 60]), torch.float32))
    with pytest.raises(ValueError):
        Int4KVMemoryManager(8, torch.float32, 2, 32, 1, torch.device("cpu"), group_size=5)

    a = LLM(config=CFG, **KW).model
    b = LLM(config=CFG, kv_type="int4kv", kv_quant_group_size=8, **KW).model
    assert isinstance(b.mem_manager, Int4KVMemoryManager) and b.kv_bytes_per_token() == 2 * 2 * 2 * (8 + 4)
    ids = torch.randint(3, 300, (50,), generator=torch.Generator().manual_seed(3))

    def run(m):
        req = m.req_manager.alloc()
        mi = ModelInput(batch_size=1, total_token_num=50, max_kv_len=50, is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([50], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(50).clone(), input_ids=ids,
                        b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=50, return_all_logits=True)
        out = [m.forward(mi).logits.float()]
        m.req_manager.req_to_next_token_ids[req] = 17
        mi = ModelInput(batch_size=1, total_token_num=51, max_kv_len=51, is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([51], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(1).clone())
        out.append(m.forward(mi).logits.float())
        return torch.cat(out)

    la, lb = run(a), run(b)
    scale = la.abs().max().item()
    assert (la - lb).abs().max().item() < 0.25 * scale               # 4-bit rows: about 7 % per element
    assert (la.argmax(-1) == lb.argmax(-1)).float().mean() > 0.6
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 300, n).tolist() for n in (9, 40, 70)]
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    llm = LLM(config=CFG, kv_type="int4kv", **KW)
    out = llm.generate(prompts, sp)
    again = llm.generate(prompts, sp)
    assert all(len(o["token_ids"]) == 8 for o in out) and again[2]["prompt_cache_len"] > 0
