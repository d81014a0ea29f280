"""Prefix reuse for hybrid (linear-attention) models: snapshots of the recurrent state at page boundaries.

A request of a hybrid model can only continue from a cached prefix if, besides the KV of the full-attention layers
(the radix tree), the convolution / matrix state of every linear-attention layer *at the end of that prefix* is
known.  The model keeps a small table of state snapshots; this index maps "the first L tokens" (L a multiple of the
page size, keyed by a hash chain over the pages) to a snapshot slot, least recently used slots are overwritten.

* save: after a prefill chunk or a decode step that leaves a request at a page boundary;
* lookup: for a new request whose radix match covers n tokens, the longest snapshotted boundary L <= n of its
  own prompt; the match is trimmed to L and the snapshot is copied into the request's state rows.

The scheduler ends a prefill chunk at the last page boundary of the prompt, so a finished conversation leaves a
snapshot that the next turn (same tokens + more) can start from.

Snapshots are large (every linear layer's matrix state), so the table on the GPU is small.  With a host tier
(`host_bytes > 0`: `--enable_cpu_cache` without `--disable_linear_att_small_page_cpu_cache`) a snapshot that falls out
of the GPU table moves to pinned host memory instead of being lost, and a lookup that finds it there brings it back
into a GPU slot; the host tier evicts least recently used entries for good.

Reference: lightllm/server/router/dynamic_prompt/linear_att_radix_cache.py (hash-paged tree nodes carrying
linear-attention buffers), lightllm/common/linear_att_cache_manager/.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from typing import List, Optional, Tuple

import numpy as np


def page_hash_chain(ids: np.ndarray, page: int, n_pages: Optional[int] = None) -> List[bytes]:
    """keys[i] identifies tokens [0, (i + 1) * page)."""
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    total = len(ids) // page if n_pages is None else min(n_pages, len(ids) // page)
    out, h = [], b""
    for p in range(total):
        h = hashlib.blake2b(h + ids[p * page:(p + 1) * page].tobytes(), digest_size=16).digest()
        out.append(h)
    return out


class StateSnapshotCache:
    def __init__(self, model, page: int, host_bytes: int = 0):
        self.model = model
        self.page = int(page)
        self.n_slots = int(model.state_snapshot_slots)
        assert self.n_slots > 0 and self.page > 0
        self.index: "OrderedDict[bytes, Tuple[int, int]]" = OrderedDict()   # key -> (slot, length); LRU order
        self.free = list(range(self.n_slots - 1, -1, -1))
        self.stats = {"saved": 0, "hits": 0, "hit_tokens": 0, "evicted": 0, "to_host": 0, "from_host": 0}
        # host tier: key -> (host slot, length)
        self.host_index: "OrderedDict[bytes, Tuple[int, int]]" = OrderedDict()
        self.host_slots = 0
        if host_bytes > 0 and hasattr(model, "alloc_host_snapshots"):
            self.host_slots = int(model.alloc_host_snapshots(int(host_bytes)))
        self.host_free = list(range(self.host_slots - 1, -1, -1))

    def __len__(self):
        return len(self.index)

    def _gpu_slot(self) -> int:
        """A free slot of the GPU table; the least recently used snapshot moves to the host tier (or is dropped)."""
        if not self.free:
            key, (slot, length) = self.index.popitem(last=False)
            self.stats["evicted"] += 1
            if self.host_slots > 0:
                if not self.host_free:
                    _, (h, _) = self.host_index.popitem(last=False)
                    self.host_free.append(h)
                h = self.host_free.pop()
                self.model.export_state_snapshot(slot, h)
                self.host_index[key] = (h, length)
                self.stats["to_host"] += 1
            self.free.append(slot)
        return self.free.pop()

    def save(self, req_idx: int, ids: np.ndarray) -> bool:
        """Snapshot of request `req_idx` whose state covers exactly `ids` (length a multiple of the page)."""
        L = len(ids)
        if L == 0 or L % self.page:
            return False
        key = page_hash_chain(ids, self.page)[-1]
        hit = self.index.get(key)
        if hit is not None:          # same prefix already kept: refresh its age
            self.index.move_to_end(key)
            return False
        stale = self.host_index.pop(key, None)     # the fresh copy on the GPU replaces a host copy
        if stale is not None:
            self.host_free.append(stale[0])
        slot = self._gpu_slot()
        self.model.save_state_snapshot(slot, req_idx)
        self.index[key] = (slot, L)
        self.stats["saved"] += 1
        return True

    def lookup(self, ids: np.ndarray, max_len: int) -> Tuple[int, Optional[int]]:
        """(L, slot) of the longest snapshot of a prefix of `ids` with L <= max_len; (0, None) without one.  A
        snapshot found in the host tier is brought into a GPU slot first."""
        n_pages = min(max_len, len(ids)) // self.page
        if n_pages <= 0 or not (self.index or self.host_index):
            return 0, None
        keys = page_hash_chain(ids, self.page, n_pages)
        for p in range(n_pages - 1, -1, -1):
            k = keys[p]
            hit = self.index.get(k)
            if hit is not None:
                self.index.move_to_end(k)
                return (p + 1) * self.page, hit[0]
            on_host = self.host_index.pop(k, None)
            if on_host is not None:
                h, length = on_host
                slot = self._gpu_slot()       # may push another snapshot out to the host tier (not into `h`: it
                self.model.import_state_snapshot(h, slot)   # is not free yet)
                self.host_free.append(h)
                self.index[k] = (slot, length)
                self.stats["from_host"] += 1
                return length, slot
        return 0, None

    def restore(self, slot: int, req_idx: int, length: int):
        self.model.load_state_snapshot(slot, req_idx)
        self.stats["hits"] += 1
        self.stats["hit_tokens"] += length

    def clear(self):
        self.index.clear()
        self.free = list(range(self.n_slots - 1, -1, -1))
        self.host_index.clear()
        self.host_free = list(range(self.host_slots - 1, -1, -1))
