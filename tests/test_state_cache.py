"""Prefix reuse for hybrid (Gated DeltaNet) models through recurrent-state snapshots: a follow-up request that
shares a long prefix starts from the snapshot and produces exactly what it produces without any cache."""
import numpy as np
import torch

from lightllm_b200.engine.llm import LLM
from lightllm_b200.engine.state_cache import StateSnapshotCache, page_hash_chain

CFG = dict(model_type="qwen3_5_text", hidden_size=64, intermediate_size=128, num_hidden_layers=4,
           num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=300, rms_norm_eps=1e-6,
           linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
           linear_conv_kernel_dim=4, full_attention_interval=4, max_position_embeddings=512, eos_token_id=2,
           tie_word_embeddings=False)
KW = dict(max_total_token_num=4096, running_max_req_size=8, max_req_total_len=512, batch_max_tokens=256,
          data_type="float32")


def test_hash_chain_and_lru_index():
    ids = np.arange(100)
    a = page_hash_chain(ids, 16)
    assert len(a) == 6 and page_hash_chain(ids[:40], 16) == a[:2]
    other = ids.copy()
    other[3] = 7
    assert page_hash_chain(other, 16)[0] != a[0]

    class M:
        state_snapshot_slots = 2

        def __init__(self):
            self.saved, self.loaded = [], []

        def save_state_snapshot(self, slot, req):
            self.saved.append((slot, req))

        def load_state_snapshot(self, slot, req):
            self.loaded.append((slot, req))

    m = M()
    c = StateSnapshotCache(m, 16)
    assert not c.save(0, ids[:20])                       # not at a page boundary
    assert c.save(0, ids[:32]) and c.save(1, ids[:64]) and not c.save(1, ids[:64])
    assert c.lookup(ids, 100)[0] == 64 and c.lookup(ids, 63)[0] == 32 and c.lookup(ids, 31) == (0, None)
    assert c.lookup(other, 100) == (0, None)
    c.lookup(ids, 40)                                    # touches the 32-token snapshot: 64 is now the oldest
    assert c.save(2, other[:16]) and c.stats["evicted"] == 1
    assert c.lookup(ids, 100)[0] == 32


def test_followup_request_starts_from_a_snapshot():
    rng = np.random.default_rng(0)
    first = rng.integers(3, 300, 150).tolist()
    sp = {"max_new_tokens": 20, "ignore_eos": True}
    plain = LLM(config=CFG, **KW)
    assert plain.backend.radix_cache is None            # no snapshots: the prefix cache stays off
    out1 = plain.generate([first], sp)[0]["token_ids"]
    turn2 = first + out1 + rng.integers(3, 300, 30).tolist()
    want2 = plain.generate([turn2], sp)[0]["token_ids"]

    llm = LLM(config=CFG, state_snapshot_slots=4, linear_att_hash_page_size=32, **KW)
    sc = llm.backend.state_cache
    assert sc is not None and llm.backend.radix_cache is not None
    got1 = llm.generate([first], sp)[0]["token_ids"]
    assert got1 == out1
    # snapshots: the last page boundary of the prompt (128) and the boundary crossed while decoding (160)
    assert sc.stats["saved"] == 2 and sc.stats["hits"] == 0
    got2 = llm.generate([turn2], sp)[0]["token_ids"]
    assert got2 == want2
    assert sc.stats["hits"] == 1 and sc.stats["hit_tokens"] == 160    # 170 tokens were in the tree, 160 had a state
    # an unrelated prompt takes nothing from the cache
    other = rng.integers(3, 300, 90).tolist()
    assert llm.generate([other], sp)[0]["token_ids"] == plain.generate([other], sp)[0]["token_ids"]
    assert sc.stats["hits"] == 1
    # nothing leaked
    rc = llm.backend.radix_cache
    assert llm.model.mem_manager.can_use_mem_size + rc.get_tree_total_tokens_num() == llm.model.mem_manager.size
    assert rc.get_refed_tokens_num() == 0


def test_concurrent_requests_with_a_shared_system_prompt():
    rng = np.random.default_rng(1)
    system = rng.integers(3, 300, 100).tolist()
    prompts = [system + rng.integers(3, 300, n).tolist() for n in (20, 45, 7)]
    sp = {"max_new_tokens": 10, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=CFG, **KW).generate(prompts, sp)]
    llm = LLM(config=CFG, state_snapshot_slots=8, linear_att_hash_page_size=32, **KW)
    assert [o["token_ids"] for o in llm.generate(prompts[:1], sp)] == want[:1]     # leaves a snapshot at 96
    got = [o["token_ids"] for o in llm.generate(prompts, sp)]
    assert got == want
    assert llm.backend.state_cache.stats["hits"] >= 3


def test_recurrent_state_kept_in_bf16():
    rng = np.random.default_rng(4)
    prompts = [rng.integers(3, 300, n).tolist() for n in (40, 70)]
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=CFG, **KW).generate(prompts, sp)]
    llm = LLM(config=CFG, linear_att_ssm_data_type="bfloat16", state_snapshot_slots=2, linear_att_hash_page_size=32, **KW)
    assert llm.model.ssm_state.dtype == torch.bfloat16 and llm.model.ssm_snap.dtype == torch.bfloat16
    got = [o["token_ids"] for o in llm.generate(prompts, sp)]
    same = sum(a == b for x, y in zip(want, got) for a, b in zip(x, y))
    assert same >= 12          # bf16 state: nearly the same greedy tokens on this toy model


def test_host_tier_keeps_snapshots_that_fall_out_of_the_gpu_table():
    ids = np.arange(200)

    class M:
        state_snapshot_slots = 1

        def __init__(self):
            self.gpu, self.host, self.req_state = {}, {}, {}

        def save_state_snapshot(self, slot, req):
            self.gpu[slot] = self.req_state[req]

        def load_state_snapshot(self, slot, req):
            self.req_state[req] = self.gpu[slot]

        def alloc_host_snapshots(self, nbytes):
            return nbytes // 100

        def export_state_snapshot(self, slot, h):
            self.host[h] = self.gpu[slot]

        def import_state_snapshot(self, h, slot):
            self.gpu[slot] = self.host[h]

    m = M()
    c = StateSnapshotCache(m, 16, host_bytes=250)       # one GPU slot, two host slots
    assert c.host_slots == 2
    m.req_state = {0: "s32", 1: "s64", 2: "s96", 3: "s128"}
    assert c.save(0, ids[:32]) and c.save(1, ids[:64])               # 32 moves to the host
    assert c.stats["to_host"] == 1 and [v[1] for v in c.host_index.values()] == [32]
    assert c.lookup(ids, 63) == (32, 0)                              # found on the host, back in the GPU slot;
    assert c.stats["from_host"] == 1 and m.gpu[0] == "s32"           # 64 took its place on the host
    assert [v[1] for v in c.host_index.values()] == [64]
    c.restore(0, 7, 32)
    assert m.req_state[7] == "s32"
    assert c.save(2, ids[:96]) and c.save(3, ids[:128])              # host: 64, 32, then 96 pushes 64 out for good
    assert sorted(v[1] for v in c.host_index.values()) == [32, 96]
    assert c.lookup(ids, 80) == (32, 0) and m.gpu[0] == "s32"        # 64 is gone, 32 is the longest left below 80
    assert c.lookup(ids, 200)[0] == 128                              # (now on the host) comes back
    m.req_state[4] = "s128b"
    assert not c.save(4, ids[:128])                                  # already on the GPU: only refreshed
    c.clear()
    assert c.lookup(ids, 200) == (0, None) and len(c.host_free) == 2


def test_second_turn_starts_from_a_snapshot_kept_on_the_host():
    rng = np.random.default_rng(3)
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    a = rng.integers(3, 300, 100).tolist()
    b = rng.integers(3, 300, 100).tolist()
    plain = LLM(config=CFG, **KW)
    a2 = a + plain.generate([a], sp)[0]["token_ids"] + rng.integers(3, 300, 20).tolist()
    want = plain.generate([a2], sp)[0]["token_ids"]

    llm = LLM(config=CFG, state_snapshot_slots=1, linear_att_hash_page_size=32, state_host_cache_bytes=8 << 20, **KW)
    sc = llm.backend.state_cache
    assert sc.host_slots > 1
    llm.generate([a], sp)
    llm.generate([b], sp)             # the only GPU slot now holds a snapshot of b
    assert sc.stats["to_host"] >= 1
    got = llm.generate([a2], sp)[0]
    assert got["token_ids"] == want and sc.stats["from_host"] == 1 and sc.stats["hits"] == 1
    assert got["prompt_cache_len"] == 96       # the prompt's last boundary (decoding 8 tokens crossed no other one)
