"""Radix prefix cache over token ids; values are KV pool slot indices.

Finished requests donate their KV to the tree; a new request whose prompt shares a prefix
with a cached path reuses those slots (the prefill only computes the remainder).  Nodes are
reference counted while a running request uses them; eviction removes unreferenced leaves,
oldest first, and hands their slots back to the pool.

Behavioural counterpart: lightllm/server/router/dynamic_prompt/radix_cache.py:101-510.
The token-matching inner loops run on numpy arrays (vectorised compare), the node ordering for
eviction is a heap keyed by last-access time.
"""
from __future__ import annotations

import heapq
import itertools
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np


def _match_len(a: np.ndarray, b: np.ndarray) -> int:
    n = min(a.shape[0], b.shape[0])
    if n == 0:
        return 0
    neq = np.flatnonzero(a[:n] != b[:n])
    return int(neq[0]) if neq.size else n


class TreeNode:
    __slots__ = ("children", "parent", "key", "value", "ref_counter", "time_id", "node_len", "_alive")

    def __init__(self):
        self.children: Dict[int, "TreeNode"] = {}
        self.parent: Optional["TreeNode"] = None
        self.key: np.ndarray = np.empty(0, dtype=np.int64)
        self.value: np.ndarray = np.empty(0, dtype=np.int32)
        self.ref_counter = 0
        self.time_id = 0
        self.node_len = 0
        self._alive = True

    def is_leaf(self) -> bool:
        return not self.children

    def __lt__(self, other):  # heap tie-break
        return self.time_id < other.time_id


class RadixCache:
    def __init__(self, unique_name: str = "radix", total_token_num: int = 0, rank_in_node: int = 0, mem_manager=None,
                 shared_counters=None):
        self.mem_manager = mem_manager
        self.root = TreeNode()
        self.root.ref_counter = 1  # never evicted
        self._tick = itertools.count(1)
        self.tree_total_tokens_num = 0
        self.refed_tokens_num = 0
        self._evict_heap: List[Tuple[int, int, TreeNode]] = []
        self._shared = shared_counters  # optional object with .set(refed, total) mirrored to shm for the router
        self._seq = itertools.count()

    # ---- bookkeeping ----
    def _touch(self, node: TreeNode):
        node.time_id = next(self._tick)

    def _publish(self):
        if self._shared is not None:
            self._shared.set(self.refed_tokens_num, self.tree_total_tokens_num)

    def _maybe_evictable(self, node: TreeNode):
        if node is not self.root and node.ref_counter == 0 and node.is_leaf() and node._alive:
            heapq.heappush(self._evict_heap, (node.time_id, next(self._seq), node))

    def get_refed_tokens_num(self) -> int:
        return self.refed_tokens_num

    def get_tree_total_tokens_num(self) -> int:
        return self.tree_total_tokens_num

    def unreferenced_tokens_num(self) -> int:
        return self.tree_total_tokens_num - self.refed_tokens_num

    # ---- core ops ----
    def _split(self, node: TreeNode, at: int) -> TreeNode:
        """Split `node` so that its first `at` tokens become a new parent; returns that parent."""
        head = TreeNode()
        head.key, head.value = node.key[:at], node.value[:at]
        head.node_len = at
        head.parent = node.parent
        head.ref_counter = node.ref_counter
        head.time_id = node.time_id
        node.parent.children[int(head.key[0])] = head
        node.key, node.value = node.key[at:], node.value[at:]
        node.node_len = node.key.shape[0]
        node.parent = head
        head.children[int(node.key[0])] = node
        return head

    def insert(self, key: np.ndarray, value: np.ndarray) -> int:
        """Adds the path; returns how many leading tokens were already present (their new slots are
        duplicates the caller must free)."""
        key = np.asarray(key, dtype=np.int64)
        value = np.asarray(value, dtype=np.int32)
        assert key.shape[0] == value.shape[0]
        node = self.root
        pos = 0
        n = key.shape[0]
        self._touch(node)
        while pos < n:
            child = node.children.get(int(key[pos]))
            if child is None:
                new = TreeNode()
                new.key, new.value = key[pos:].copy(), value[pos:].copy()
                new.node_len = n - pos
                new.parent = node
                node.children[int(key[pos])] = new
                self._touch(new)
                self.tree_total_tokens_num += new.node_len
                self._maybe_evictable(new)
                self._publish()
                return pos
            m = _match_len(child.key, key[pos:])
            if m < child.node_len:
                child = self._split(child, m)
            self._touch(child)
            pos += m
            node = child
        self._publish()
        return pos

    def match_prefix(self, key: np.ndarray, update_refs: bool = False):
        """Longest cached prefix of `key`: (last node, length, slot array) or (None, 0, None)."""
        key = np.asarray(key, dtype=np.int64)
        node = self.root
        pos = 0
        n = key.shape[0]
        values = []
        while pos < n:
            child = node.children.get(int(key[pos]))
            if child is None:
                break
            m = _match_len(child.key, key[pos:])
            if m == 0:
                break
            if m < child.node_len:
                child = self._split(child, m)
            values.append(child.value)
            self._touch(child)
            pos += m
            node = child
            if m < child.node_len:
                break
        if pos == 0:
            return None, 0, None
        if update_refs:
            self.add_node_ref_counter(node)
        return node, pos, np.concatenate(values) if len(values) > 1 else values[0].copy()

    def add_node_ref_counter(self, node: Optional[TreeNode]):
        while node is not None and node is not self.root:
            if node.ref_counter == 0:
                self.refed_tokens_num += node.node_len
            node.ref_counter += 1
            node = node.parent
        self._publish()

    def dec_node_ref_counter(self, node: Optional[TreeNode]):
        while node is not None and node is not self.root:
            node.ref_counter -= 1
            assert node.ref_counter >= 0
            if node.ref_counter == 0:
                self.refed_tokens_num -= node.node_len
                self._maybe_evictable(node)
            node = node.parent
        self._publish()

    def evict(self, need_remove_tokens: int, evict_callback: Callable[[np.ndarray], None]) -> int:
        """Removes unreferenced leaves (least recently used first) until `need_remove_tokens` slots were
        released; returns the number released."""
        released = 0
        while released < need_remove_tokens and self._evict_heap:
            t, _, node = heapq.heappop(self._evict_heap)
            if not node._alive or node.ref_counter != 0 or not node.is_leaf() or t != node.time_id:
                if node._alive and node.ref_counter == 0 and node.is_leaf() and t != node.time_id:
                    heapq.heappush(self._evict_heap, (node.time_id, next(self._seq), node))  # stale timestamp
                continue
            evict_callback(node.value)
            released += node.node_len
            self.tree_total_tokens_num -= node.node_len
            parent = node.parent
            del parent.children[int(node.key[0])]
            node._alive = False
            self._maybe_evictable(parent)
        self._publish()
        return released

    def free_radix_cache_to_get_enough_token(self, need_token_num: int):
        """Evict until the pool can serve `need_token_num` slots (no-op if it already can)."""
        if self.mem_manager is None:
            return
        free = self.mem_manager.can_use_mem_size
        if need_token_num > free:
            missing = need_token_num - free
            chunks = []
            self.evict(missing, lambda v: chunks.append(v))
            if chunks:
                self.mem_manager.free(np.concatenate(chunks))

    def publish(self, key, slots) -> int:
        """Insert externally filled slots; spare copies of already present positions go back to the pool."""
        v = np.asarray(slots.cpu() if hasattr(slots, "cpu") else slots, dtype=np.int32)
        k = np.asarray(key.cpu() if hasattr(key, "cpu") else key, dtype=np.int64)
        present = self.insert(k, v)
        if present and self.mem_manager is not None:
            self.mem_manager.free(v[:present])
        return present

    def clear_tree_nodes(self):
        """Drop every unreferenced path (flush_cache)."""
        chunks = []
        self.evict(self.tree_total_tokens_num, lambda v: chunks.append(v))
        if chunks and self.mem_manager is not None:
            self.mem_manager.free(np.concatenate(chunks))

    def merge_unreferenced_nodes(self):
        """Compaction: an unreferenced node whose only child is unreferenced too absorbs that child.  Handles that
        callers hold always have a reference count above zero, so none is invalidated.  Returns the number of
        nodes merged away.  Reference: dynamic_prompt/radix_cache.py:347-403."""
        merged = 0
        stack = [self.root]
        while stack:
            node = stack.pop()
            for child in list(node.children.values()):
                while len(child.children) == 1 and child.ref_counter == 0:
                    (gc,) = child.children.values()
                    if gc.ref_counter != 0:
                        break
                    merged += 1
                    child.key = np.concatenate([child.key, gc.key])
                    child.value = np.concatenate([child.value, gc.value])
                    child.node_len = child.key.shape[0]
                    child.children = gc.children
                    for c in child.children.values():
                        c.parent = child
                    child.time_id = max(child.time_id, gc.time_id)
                    gc._alive = False
                    self._maybe_evictable(child)
                stack.append(child)
        return merged

    def all_nodes(self):
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            out.append(n)
            stack.extend(n.children.values())
        return out
