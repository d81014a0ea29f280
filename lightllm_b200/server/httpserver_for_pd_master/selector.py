"""(P, D) node selection policies of the pd_master: random, round_robin, adaptive_load (importance
sampling on free KV capacity) and cache_aware (prefix affinity for the prefill node, bounded by load).
Reference: lightllm/server/httpserver_for_pd_master/pd_selector/{pd_selector,cache_aware,prompt_cache_tree}.py.
"""
from __future__ import annotations

import random
import time
from typing import Dict, List, Optional, Tuple

from ..pd_io_struct import PDClient


class PDSelector:
    def __init__(self):
        self.prefill_nodes: List[PDClient] = []
        self.decode_nodes: List[PDClient] = []

    def update_nodes(self, prefill_nodes, decode_nodes):
        self.prefill_nodes, self.decode_nodes = list(prefill_nodes), list(decode_nodes)

    def select_p_d_node(self, prompt, sampling_params=None, multimodal_params=None) -> Tuple[PDClient, PDClient]:
        raise NotImplementedError

    def record_prompt_cache_hit_rate(self, rate: float):
        pass

    def forget_node(self, node: PDClient):
        pass


class RandomSelector(PDSelector):
    def select_p_d_node(self, prompt, sampling_params=None, multimodal_params=None):
        return random.choice(self.prefill_nodes), random.choice(self.decode_nodes)


class RoundRobinSelector(PDSelector):
    def __init__(self):
        super().__init__()
        self._p = self._d = 0

    def select_p_d_node(self, prompt, sampling_params=None, multimodal_params=None):
        p = self.prefill_nodes[self._p % len(self.prefill_nodes)]
        d = self.decode_nodes[self._d % len(self.decode_nodes)]
        self._p, self._d = self._p + 1, self._d + 1
        return p, d


def _by_free_capacity(nodes: List[PDClient]) -> PDClient:
    w = [max(1.0 - n.run_status.total_token_usage_rate, 0.02) for n in nodes]
    return random.choices(nodes, weights=w)[0]


class AdaptiveLoadSelector(PDSelector):
    def select_p_d_node(self, prompt, sampling_params=None, multimodal_params=None):
        return _by_free_capacity(self.prefill_nodes), _by_free_capacity(self.decode_nodes)


class _TrieNode:
    __slots__ = ("children", "owners", "parent", "key", "stamp")

    def __init__(self, parent=None, key=None):
        self.children: Dict[str, "_TrieNode"] = {}
        self.owners: Dict[str, float] = {}  # node address -> last use
        self.parent, self.key, self.stamp = parent, key, time.monotonic()


class SampledPrefixIndex:
    """Which prefill node has seen which prompt prefix.  A prompt is thinned to one character every
    `stride` characters (so a 100k-character prompt is a path of ~200 nodes), the path is stored in a trie
    whose nodes remember the workers that served them; `match` returns, per worker, how many original
    characters of the prompt's prefix that worker has seen.  Leaves are dropped oldest-first over a size cap."""

    def __init__(self, stride: int = 512, max_nodes: int = 1_000_000, evict_batch: int = 10_000):
        self.stride, self.max_nodes, self.evict_batch = stride, max_nodes, evict_batch
        self.root = _TrieNode()
        self.size = 0

    def _keys(self, text: str):
        return [text[i] for i in range(self.stride - 1, len(text), self.stride)]

    def insert(self, text: str, owner: str):
        node, now = self.root, time.monotonic()
        for k in self._keys(text):
            nxt = node.children.get(k)
            if nxt is None:
                nxt = node.children[k] = _TrieNode(node, k)
                self.size += 1
            nxt.owners[owner] = now
            nxt.stamp = now
            node = nxt
        if self.size > self.max_nodes:
            self.evict(self.evict_batch)

    def match(self, text: str) -> Dict[str, int]:
        """owner -> matched characters (a multiple of stride)."""
        best: Dict[str, int] = {}
        node, depth = self.root, 0
        for k in self._keys(text):
            node = node.children.get(k)
            if node is None:
                break
            depth += 1
            for o in node.owners:
                best[o] = depth * self.stride
        return best

    def evict(self, n: int):
        leaves = []
        stack = [self.root]
        while stack:
            x = stack.pop()
            if not x.children and x is not self.root:
                leaves.append(x)
            stack.extend(x.children.values())
        leaves.sort(key=lambda x: x.stamp)
        for leaf in leaves[:n]:
            del leaf.parent.children[leaf.key]
            self.size -= 1

    def remove_owner(self, owner: str):
        stack = [self.root]
        while stack:
            x = stack.pop()
            x.owners.pop(owner, None)
            stack.extend(x.children.values())


class CacheAwareSelector(AdaptiveLoadSelector):
    """Prefill node: an idle node first (no GPU sits unused); else the node that has seen the longest
    prefix of this prompt if that covers more than `cache_threshold` of it and its in-flight prompt volume is
    within `balance_rel_threshold` x the least loaded node's; else the least loaded.  The load bound is
    adapted from the prompt-cache hit rate the nodes report: when a window's mean hit rate falls versus
    the previous window, affinity is favoured (bound up), when it rises the bound tightens back.
    The decode node is chosen by free capacity."""

    def __init__(self, cache_threshold=0.5, balance_rel_threshold=1.5, lo=1.0, hi=2.0, step=0.05, window=1000,
                 stride=512):
        super().__init__()
        self.cache_threshold = cache_threshold
        self.balance_rel_threshold, self.lo, self.hi, self.step, self.window = balance_rel_threshold, lo, hi, step, window
        self.index = SampledPrefixIndex(stride=stride)
        self._rates: List[float] = []
        self._last_mean: Optional[float] = None

    def record_prompt_cache_hit_rate(self, rate: float):
        self._rates.append(min(max(rate, 0.0), 1.0))
        if len(self._rates) < self.window:
            return
        mean = sum(self._rates) / len(self._rates)
        self._rates.clear()
        if self._last_mean is not None:
            if mean < self._last_mean:
                self.balance_rel_threshold = min(self.hi, self.balance_rel_threshold + self.step)
            elif mean > self._last_mean:
                self.balance_rel_threshold = max(self.lo, self.balance_rel_threshold - self.step)
        self._last_mean = mean

    def forget_node(self, node: PDClient):
        self.index.remove_owner(node.client_ip_port)

    def select_prefill(self, prompt: str) -> PDClient:
        nodes = self.prefill_nodes
        idle = [n for n in nodes if n.dispatched_req_num == 0]
        least = min(nodes, key=lambda n: n.dispatched_prompt_chars)
        chosen = None
        if idle:
            chosen = idle[0]
            hits = self.index.match(prompt)
            for n in idle:  # among idle nodes prefer one with the prefix
                if hits.get(n.client_ip_port, 0) > hits.get(chosen.client_ip_port, 0):
                    chosen = n
        else:
            hits = self.index.match(prompt)
            by_addr = {n.client_ip_port: n for n in nodes}
            cand = [(c, by_addr[a]) for a, c in hits.items() if a in by_addr]
            if cand:
                chars, node = max(cand, key=lambda t: t[0])
                if chars / max(len(prompt), 1) > self.cache_threshold and \
                        node.dispatched_prompt_chars <= self.balance_rel_threshold * max(least.dispatched_prompt_chars, 1):
                    chosen = node
            if chosen is None:
                chosen = least
        self.index.insert(prompt, chosen.client_ip_port)
        return chosen

    def select_p_d_node(self, prompt, sampling_params=None, multimodal_params=None):
        if not isinstance(prompt, str):
            prompt = "".join(chr(0x100 + (int(t) & 0xFFFF)) for t in prompt)  # token ids: one char per token
        return self.select_prefill(prompt), _by_free_capacity(self.decode_nodes)


def create_selector(name: str) -> PDSelector:
    table = {"random": RandomSelector, "round_robin": RoundRobinSelector, "adaptive_load": AdaptiveLoadSelector,
             "cache_aware": CacheAwareSelector}
    if name not in table:
        raise ValueError(f"unknown --select_p_d_node_strategy {name}; choose from {sorted(table)}")
    return table[name]()
