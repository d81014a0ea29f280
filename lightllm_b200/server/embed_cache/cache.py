"""Embedding cache for images and audio: content-hash keyed records with reference counts, a shared
embedding arena and virtual token-id ranges.

A record owns (a) a run of `token_num` virtual token ids starting at `token_id` (>= 100,000,000, above any
vocabulary; the LLM recognises them in the prompt and reads embeddings instead of the word table; equal
content gets equal ids, so the prefix cache works across requests that share an image) and (b) `token_num`
rows of the arena `[rows, hidden]` in POSIX shared memory, written by the visual/audio server and read by every
LLM rank.  Records with ref == 0 are evicted least-recently-used first when capacity or arena rows run out.
Reference: lightllm/server/embed_cache/impl/naive_memory_cache.py, allocator.py, embed_cache_client.py.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from multiprocessing import shared_memory
from typing import Dict, List, Optional, Tuple

import numpy as np

TOKEN_ID_BASE = 100_000_000


class RowAllocator:
    """First-fit allocator of contiguous row runs with coalescing free list."""

    def __init__(self, rows: int):
        self.rows = rows
        self.free: List[Tuple[int, int]] = [(0, rows)]  # sorted (start, length)

    def alloc(self, n: int) -> Optional[int]:
        for i, (s, ln) in enumerate(self.free):
            if ln >= n:
                if ln == n:
                    self.free.pop(i)
                else:
                    self.free[i] = (s + n, ln - n)
                return s
        return None

    def release(self, start: int, n: int):
        import bisect

        i = bisect.bisect_left(self.free, (start, 0))
        self.free.insert(i, (start, n))
        if i + 1 < len(self.free) and self.free[i][0] + self.free[i][1] == self.free[i + 1][0]:
            self.free[i] = (self.free[i][0], self.free[i][1] + self.free[i + 1][1])
            self.free.pop(i + 1)
        if i > 0 and self.free[i - 1][0] + self.free[i - 1][1] == self.free[i][0]:
            self.free[i - 1] = (self.free[i - 1][0], self.free[i - 1][1] + self.free[i][1])
            self.free.pop(i)

    def free_rows(self) -> int:
        return sum(ln for _, ln in self.free)


class EmbedArena:
    """[rows, hidden] uint16 (bf16 bit patterns) in shared memory."""

    def __init__(self, name: str, rows: int, hidden: int, create: bool):
        self.rows, self.hidden = rows, hidden
        nbytes = rows * hidden * 2
        if create:
            try:
                old = shared_memory.SharedMemory(name=name)
                old.close()
                old.unlink()
            except FileNotFoundError:
                pass
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=nbytes)
        else:
            self.shm = shared_memory.SharedMemory(name=name)
        self.arr = np.ndarray((rows, hidden), dtype=np.uint16, buffer=self.shm.buf)
        self._owner = create

    def write(self, start: int, emb) -> None:
        """emb: torch bf16/float tensor or uint16 array [n, hidden]."""
        import torch

        if isinstance(emb, torch.Tensor):
            emb = emb.detach().to(torch.bfloat16).cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
        self.arr[start:start + emb.shape[0]] = emb

    def read_torch(self, start: int, n: int):
        import torch

        return torch.from_numpy(self.arr[start:start + n].view(np.int16)).view(torch.bfloat16)

    def read_rows(self, rows):
        """Arbitrary rows (int64 tensor) as a bf16 tensor."""
        import torch

        idx = rows.cpu().numpy() if hasattr(rows, "cpu") else np.asarray(rows)
        return torch.from_numpy(self.arr[idx].view(np.int16)).view(torch.bfloat16)

    def close(self):
        self.arr = None
        self.shm.close()
        if self._owner:
            try:
                self.shm.unlink()
            except FileNotFoundError:
                pass


@dataclass
class Record:
    id: int
    md5: str
    ref: int
    data: bool
    embed: bool
    created: float
    visited: float
    token_id: int
    token_num: int
    row_start: int
    payload: Optional[bytes] = None


class EmbedCache:
    def __init__(self, capacity: int, arena_rows: int, id_range_source=None):
        self.capacity = max(1, capacity)
        self.rows = RowAllocator(arena_rows)
        self.by_id: Dict[int, Record] = {}
        self.by_md5: Dict[str, Record] = {}
        self.lock = threading.Lock()
        self._next_id = 1
        self._id_range_source = id_range_source  # callable -> (start, end), e.g. the config server
        self.token_lo, self.token_hi = (TOKEN_ID_BASE, 2 ** 63 - 1) if id_range_source is None else (0, 0)

    def _take_token_ids(self, n: int) -> int:
        if self.token_lo + n >= self.token_hi:
            self.token_lo, self.token_hi = self._id_range_source()
            assert self.token_lo + n < self.token_hi
        s = self.token_lo
        self.token_lo += n
        return s

    def _evict_one(self) -> bool:
        idle = [r for r in self.by_id.values() if r.ref <= 0]
        if not idle:
            return False
        r = min(idle, key=lambda r: (r.visited, r.id))
        self.rows.release(r.row_start, r.token_num)
        del self.by_id[r.id], self.by_md5[r.md5]
        return True

    def alloc(self, md5s: List[str], token_nums: List[int]) -> Optional[List[dict]]:
        """All-or-nothing: records for every item (existing ones get ref + 1) or None when the cache cannot make
        room (the caller retries later)."""
        now = time.time()
        with self.lock:
            uniq = {}
            for m, n in zip(md5s, token_nums):
                uniq.setdefault(m, n)
            new = [(m, n) for m, n in uniq.items() if m not in self.by_md5]
            for m in uniq:
                if m in self.by_md5:
                    self.by_md5[m].ref += 1  # pin hits so eviction below cannot take them
            ok = True
            made: List[Record] = []
            for m, n in new:
                while len(self.by_id) >= self.capacity and self._evict_one():
                    pass
                start = self.rows.alloc(n)
                while start is None and self._evict_one():
                    start = self.rows.alloc(n)
                if start is None or len(self.by_id) >= self.capacity:
                    if start is not None:
                        self.rows.release(start, n)
                    ok = False
                    break
                rec = Record(self._next_id, m, 1, False, False, now, now, self._take_token_ids(n), n, start)
                self._next_id += 1
                self.by_id[rec.id] = self.by_md5[m] = rec
                made.append(rec)
            if not ok:
                for rec in made:
                    self.rows.release(rec.row_start, rec.token_num)
                    del self.by_id[rec.id], self.by_md5[rec.md5]
                for m in uniq:
                    if m in self.by_md5:
                        self.by_md5[m].ref -= 1
                return None
            out = []
            seen = set()
            for m in md5s:
                rec = self.by_md5[m]
                if m in seen:
                    rec.ref += 1  # every occurrence holds one reference
                seen.add(m)
                rec.visited = now
                out.append({"id": rec.id, "token_id": rec.token_id, "token_num": rec.token_num,
                            "start_index_in_embed_cache": rec.row_start})
            return out

    def release(self, ids: List[int]):
        with self.lock:
            for i in ids:
                r = self.by_id.get(i)
                if r is not None:
                    r.ref -= 1

    def set_items_data(self, ids: List[int], payloads: Optional[List[bytes]] = None):
        with self.lock:
            for k, i in enumerate(ids):
                self.by_id[i].data = True
                if payloads is not None:
                    self.by_id[i].payload = payloads[k]

    def get_items_data(self, ids: List[int]) -> List[bool]:
        with self.lock:
            return [self.by_id[i].data if i in self.by_id else False for i in ids]

    def get_payload(self, i: int) -> Optional[bytes]:
        with self.lock:
            r = self.by_id.get(i)
            return None if r is None else r.payload

    def set_items_embed(self, ids: List[int]):
        with self.lock:
            for i in ids:
                self.by_id[i].embed = True
                self.by_id[i].payload = None  # raw bytes are not needed once embedded

    def get_items_embed(self, ids: List[int]) -> List[bool]:
        with self.lock:
            return [self.by_id[i].embed if i in self.by_id else False for i in ids]
