"""Prefix tree: hand-made invariants on both implementations (the Python specification `RadixCache` and the C++
tree behind `NativeRadixCache` that the engine uses) and a randomized differential run of the two.
Invariants follow unit_tests/server/router/dynamic_prompt/test_radix_cache.py of the reference (shared prefixes
split nodes, references pin paths, eviction takes unreferenced leaves oldest first, merge only along
single-child chains of equal reference count, flush drops everything unreferenced)."""
import numpy as np
import pytest

from lightllm_b200.engine.native_radix import NativeRadixCache
from lightllm_b200.engine.radix_cache import RadixCache

IMPLS = [RadixCache, NativeRadixCache]


def k(*ids):
    return np.array(ids, dtype=np.int64)


def v(start, n):
    return np.arange(start, start + n, dtype=np.int32)


@pytest.mark.parametrize("cls", IMPLS)
def test_insert_match_split_and_token_counts(cls):
    t = cls("t", 100, 0)
    assert t.match_prefix(k(1, 2, 3))[1] == 0
    assert t.insert(k(0, 1, 2, 3, 4, 5, 6, 7, 8, 9), v(100, 10)) == 0
    assert t.get_tree_total_tokens_num() == 10
    # a second path sharing 5 tokens: 5 already present, 3 new
    assert t.insert(k(0, 1, 2, 3, 4, 7, 8, 9), v(200, 8)) == 5
    assert t.get_tree_total_tokens_num() == 13
    node, n, slots = t.match_prefix(k(0, 1, 2, 3, 4, 7, 8, 9, 11), update_refs=False)
    assert n == 8 and slots.tolist() == [100, 101, 102, 103, 104, 205, 206, 207]   # shared part keeps the FIRST slots
    node, n, slots = t.match_prefix(k(0, 1, 2), update_refs=False)                # ends inside a node
    assert n == 3 and slots.tolist() == [100, 101, 102]
    assert t.match_prefix(k(9, 9))[1] == 0
    assert t.insert(k(0, 1, 2, 3, 4, 5, 6, 7, 8, 9), v(300, 10)) == 10            # nothing new
    assert t.get_tree_total_tokens_num() == 13 and t.get_refed_tokens_num() == 0


@pytest.mark.parametrize("cls", IMPLS)
def test_references_pin_paths_and_eviction_is_lru_over_leaves(cls):
    t = cls("t", 100, 0)
    t.insert(k(1, 2, 3, 4), v(0, 4))          # oldest
    t.insert(k(1, 2, 7, 8, 9), v(10, 5))
    t.insert(k(5, 6), v(20, 2))               # newest
    assert t.get_tree_total_tokens_num() == 2 + 2 + 3 + 2
    node, n, _ = t.match_prefix(k(1, 2, 3, 4), update_refs=True)
    assert n == 4 and t.get_refed_tokens_num() == 4 and t.unreferenced_tokens_num() == 5
    freed = []
    assert t.evict(3, lambda s: freed.extend(np.asarray(s).tolist())) == 3
    assert sorted(freed) == [12, 13, 14]      # the unreferenced leaf that was touched before [5, 6]
    freed.clear()
    assert t.evict(100, lambda s: freed.extend(np.asarray(s).tolist())) == 2      # only [5, 6] is left to take
    assert sorted(freed) == [20, 21] and t.get_tree_total_tokens_num() == 4
    t.dec_node_ref_counter(node)
    assert t.get_refed_tokens_num() == 0
    freed.clear()
    assert t.evict(100, lambda s: freed.extend(np.asarray(s).tolist())) == 4
    assert sorted(freed) == [0, 1, 2, 3] and t.get_tree_total_tokens_num() == 0
    assert t.evict(5, lambda s: freed.append(-1)) == 0


@pytest.mark.parametrize("cls", IMPLS)
def test_reference_counts_nest_and_underflow_is_caught(cls):
    t = cls("t", 100, 0)
    t.insert(k(1, 2, 3, 4, 5, 6), v(0, 6))
    a, na, _ = t.match_prefix(k(1, 2, 3), update_refs=True)          # splits [1..6] at 3
    b, nb, _ = t.match_prefix(k(1, 2, 3, 4, 5, 6), update_refs=True)
    assert (na, nb) == (3, 6) and t.get_refed_tokens_num() == 6
    t.dec_node_ref_counter(b)
    assert t.get_refed_tokens_num() == 3                             # the head is still held by `a`
    assert t.evict(10, lambda s: None) == 3                          # only the tail can go
    t.dec_node_ref_counter(a)
    assert t.get_refed_tokens_num() == 0
    with pytest.raises(AssertionError):
        t.dec_node_ref_counter(a)


@pytest.mark.parametrize("cls", IMPLS)
def test_flush_keeps_referenced_paths(cls):
    class Pool:
        def __init__(self):
            self.freed = []
            self.can_use_mem_size = 0

        def free(self, s):
            self.freed.extend(np.asarray(s).tolist())

    pool = Pool()
    t = cls("t", 100, 0, mem_manager=pool)
    t.insert(k(1, 2, 3), v(0, 3))
    t.insert(k(4, 5), v(10, 2))
    node, _, _ = t.match_prefix(k(4, 5), update_refs=True)
    t.clear_tree_nodes()
    assert sorted(pool.freed) == [0, 1, 2] and t.get_tree_total_tokens_num() == 2
    t.dec_node_ref_counter(node)
    t.clear_tree_nodes()
    assert sorted(pool.freed) == [0, 1, 2, 10, 11] and t.get_tree_total_tokens_num() == 0
    # free_radix_cache_to_get_enough_token: evicts exactly the shortfall
    t.insert(k(7, 8, 9), v(20, 3))
    pool.can_use_mem_size = 5
    t.free_radix_cache_to_get_enough_token(4)
    assert t.get_tree_total_tokens_num() == 3
    t.free_radix_cache_to_get_enough_token(7)
    assert t.get_tree_total_tokens_num() == 0


def test_merge_rules_of_the_python_tree():
    t = RadixCache("t", 100, 0)
    t.insert(k(1, 2, 3), v(0, 3))
    t.insert(k(1, 2, 3, 4, 5), v(10, 5))          # chain A[1,2,3] -> B[4,5]
    t.insert(k(1, 2, 3, 4, 5, 6), v(20, 6))       # -> C[6]
    assert len(t.all_nodes()) == 4
    t.merge_unreferenced_nodes()                  # all unreferenced: cascades into one node
    assert len(t.all_nodes()) == 2 and t.get_tree_total_tokens_num() == 6
    _, n, slots = t.match_prefix(k(1, 2, 3, 4, 5, 6))
    assert n == 6 and slots.tolist() == [0, 1, 2, 13, 14, 25]
    # a referenced middle: no merge across a change of reference count
    t2 = RadixCache("t", 100, 0)
    t2.insert(k(1, 2), v(0, 2))
    t2.insert(k(1, 2, 3, 4), v(10, 4))
    node, _, _ = t2.match_prefix(k(1, 2), update_refs=True)
    before = len(t2.all_nodes())
    t2.merge_unreferenced_nodes()
    assert len(t2.all_nodes()) == before
    # a parent with two children is never merged
    t3 = RadixCache("t", 100, 0)
    t3.insert(k(1, 2, 3), v(0, 3))
    t3.insert(k(1, 2, 4), v(10, 3))
    before = len(t3.all_nodes())
    t3.merge_unreferenced_nodes()
    assert len(t3.all_nodes()) == before


@pytest.mark.parametrize("seed", range(6))
def test_python_and_native_trees_agree_on_random_sequences(seed):
    """Insert / match (with and without references) / release / evict in random order over a small alphabet, so that
    paths share prefixes and split often.  After every operation both trees report the same return value, the same
    slots for a match, the same token totals; evictions release the same slots in the same (LRU) order."""
    rng = np.random.default_rng(seed)
    a, b = RadixCache("a", 10_000, 0), NativeRadixCache("b", 10_000, 0)
    held = []          # [(node_a, node_b)]
    next_slot = 0
    for step in range(600):
        op = rng.choice(["insert", "insert", "match", "match_ref", "release", "evict", "merge"])
        if op == "insert":
            n = int(rng.integers(1, 24))
            key = rng.integers(0, 4, size=n).astype(np.int64)
            if rng.random() < 0.5 and step > 0:   # extend something that probably exists
                key = np.concatenate([key[: n // 2], rng.integers(0, 4, size=int(rng.integers(0, 8))).astype(np.int64)])
            if key.shape[0] == 0:
                continue
            val = np.arange(next_slot, next_slot + key.shape[0], dtype=np.int32)
            next_slot += key.shape[0]
            assert a.insert(key, val) == b.insert(key, val), f"step {step}"
        elif op in ("match", "match_ref"):
            key = rng.integers(0, 4, size=int(rng.integers(1, 30))).astype(np.int64)
            ref = op == "match_ref"
            na, la, sa = a.match_prefix(key, update_refs=ref)
            nb, lb, sb = b.match_prefix(key, update_refs=ref)
            assert la == lb, f"step {step}"
            if la:
                assert np.array_equal(sa, sb), f"step {step}"
                if ref:
                    held.append((na, nb))
        elif op == "release" and held:
            na, nb = held.pop(int(rng.integers(0, len(held))))
            a.dec_node_ref_counter(na)
            b.dec_node_ref_counter(nb)
        elif op == "merge":
            assert a.merge_unreferenced_nodes() == b.merge_unreferenced_nodes(), f"step {step}"
            assert len(a.all_nodes()) == b.node_count(), f"step {step}"
        elif op == "evict":
            need = int(rng.integers(1, 40))
            fa, fb = [], []
            ra = a.evict(need, lambda s: fa.extend(np.asarray(s).tolist()))
            rb = b.evict(need, lambda s: fb.extend(np.asarray(s).tolist()))
            assert ra == rb and fa == fb, f"step {step}: {ra} {rb}"
            assert ra >= min(need, 1) or a.unreferenced_tokens_num() == 0 or ra == 0
        assert a.get_tree_total_tokens_num() == b.get_tree_total_tokens_num(), f"step {step} ({op})"
        assert a.get_refed_tokens_num() == b.get_refed_tokens_num(), f"step {step} ({op})"
        assert 0 <= a.get_refed_tokens_num() <= a.get_tree_total_tokens_num()
    for na, nb in held:
        a.dec_node_ref_counter(na)
        b.dec_node_ref_counter(nb)
    assert a.get_refed_tokens_num() == b.get_refed_tokens_num() == 0
    total = a.get_tree_total_tokens_num()
    fa, fb = [], []
    assert a.evict(10**9, lambda s: fa.extend(np.asarray(s).tolist())) == total
    assert b.evict(10**9, lambda s: fb.extend(np.asarray(s).tolist())) == total
    assert sorted(fa) == sorted(fb) and len(set(fa)) == len(fa) == total          # every slot released exactly once


def test_native_tree_compaction():
    t = NativeRadixCache("n", 100, 0)
    t.insert(k(1, 2, 3), v(0, 3))
    t.insert(k(1, 2, 3, 4, 5), v(10, 5))
    t.insert(k(1, 2, 3, 4, 5, 6), v(20, 6))
    t.insert(k(1, 2, 3, 9), v(30, 4))                   # a second branch below [1, 2, 3]
    assert t.node_count() == 5
    assert t.merge_unreferenced_nodes() == 1 and t.node_count() == 4      # [4, 5] + [6]; the fork stays
    node, n, slots = t.match_prefix(k(1, 2, 3, 4, 5, 6), update_refs=True)
    assert n == 6 and slots.tolist() == [0, 1, 2, 13, 14, 25]
    freed = []
    assert t.evict(100, lambda s: freed.extend(np.asarray(s).tolist())) == 1 and freed == [33]   # the other branch goes
    assert t.merge_unreferenced_nodes() == 0            # the remaining chain is referenced
    t.dec_node_ref_counter(node)
    assert t.merge_unreferenced_nodes() == 1 and t.node_count() == 2
    _, n, slots = t.match_prefix(k(1, 2, 3, 4, 5, 6, 7))
    assert n == 6 and slots.tolist() == [0, 1, 2, 13, 14, 25]
    assert t.insert(k(1, 2, 3, 4, 8), v(40, 5)) == 4 and t.node_count() == 4      # a merged node splits again
    assert t.evict(100, lambda s: freed.extend(np.asarray(s).tolist())) == 7 and t.get_tree_total_tokens_num() == 0


def test_backend_merges_the_tree_on_a_pass_counter(monkeypatch):
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="llama", hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2,
               head_dim=32, intermediate_size=128, vocab_size=128, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2)
    kw = dict(data_type="float32", max_total_token_num=1024, running_max_req_size=4, max_req_total_len=128, batch_max_tokens=64)
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    prompts = [list(range(3, 40)), list(range(3, 30)) + [90, 91, 92], list(range(3, 40)) + [70, 71]]
    plain = LLM(config=cfg, **kw)
    want = [plain.generate([p], sp)[0]["token_ids"] for p in prompts]
    nodes_plain = plain.backend.radix_cache.node_count() if hasattr(plain.backend.radix_cache, "node_count") else None
    monkeypatch.setenv("LIGHTLLM_RADIX_TREE_MERGE_ENABLE", "1")
    monkeypatch.setenv("LIGHTLLM_RADIX_TREE_MERGE_DELTA", "3")
    llm = LLM(config=cfg, **kw)
    assert llm.backend._merge_delta == 3
    got = [llm.generate([p], sp)[0]["token_ids"] for p in prompts]
    assert got == want and llm.backend._merge_ticks >= 18
    rc = llm.backend.radix_cache
    assert rc.get_refed_tokens_num() == 0
    assert llm.model.mem_manager.can_use_mem_size + rc.get_tree_total_tokens_num() == llm.model.mem_manager.size
    if nodes_plain is not None:
        assert rc.node_count() <= nodes_plain
