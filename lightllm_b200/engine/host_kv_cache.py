"""Second tier of the prefix cache: KV pages in pinned host memory (optionally spilling to a disk file).

When a request finishes, the full pages (`page_tokens` tokens, all layers) of its sequence that the tier does
not hold yet are copied out of the GPU pool; when a new request's prompt matches more pages here than the GPU
prefix tree holds tokens, the pages are copied into freshly allocated slots and the request starts its prefill
after them.  Pages are keyed by a hash chain over the token ids (page i's key covers tokens 0 .. (i+1)*P), kept
in LRU order; every tensor-parallel rank keeps the pages of its own KV heads and takes the same decisions,
because they only depend on the token ids.

Copy path: pool slots -> device staging page (gather kernel, main stream) -> pinned host page (async copy on a
side stream), so the inference stream never waits for PCIe; loads go the other way.
Reference: lightllm/server/multi_level_kv_cache/*, common/basemodel/triton_kernel/kv_cache_offload.py.
"""
from __future__ import annotations

import hashlib
import os
from collections import OrderedDict
from typing import List, Optional, Tuple

import numpy as np
import torch


def page_keys(ids: np.ndarray, page_tokens: int) -> List[bytes]:
    """Chained keys of the full pages of `ids`."""
    keys, h = [], b""
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    for p in range(len(ids) // page_tokens):
        h = hashlib.blake2b(h + ids[p * page_tokens:(p + 1) * page_tokens].tobytes(), digest_size=16).digest()
        keys.append(h)
    return keys


class _DiskTier:
    """Fixed-size page file with its own LRU index (pages evicted from host memory land here)."""

    def __init__(self, path: str, n_pages: int, page_shape, dtype):
        self.n_pages = n_pages
        self.page_numel = int(np.prod(page_shape))
        self.np_dtype = np.uint16 if dtype in (torch.bfloat16, torch.float16) else \
            np.int8 if dtype == torch.int8 else np.float32
        self.t_dtype = {np.uint16: torch.int16, np.int8: torch.int8, np.float32: torch.float32}[self.np_dtype]
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.mm = np.memmap(path, dtype=self.np_dtype, mode="w+", shape=(n_pages, self.page_numel))
        self.index: "OrderedDict[bytes, int]" = OrderedDict()
        self.free = list(range(n_pages - 1, -1, -1))

    def put(self, key: bytes, page: torch.Tensor):
        if key in self.index or self.n_pages == 0:
            return
        if not self.free:
            _, idx = self.index.popitem(last=False)
            self.free.append(idx)
        idx = self.free.pop()
        raw = page.contiguous().view(self.t_dtype).reshape(-1).numpy()
        self.mm[idx] = raw.view(self.np_dtype)
        self.index[key] = idx

    def get(self, key: bytes, out: torch.Tensor) -> bool:
        idx = self.index.get(key)
        if idx is None:
            return False
        self.index.move_to_end(key)
        src = torch.from_numpy(np.array(self.mm[idx])).view(self.t_dtype)
        out.view(src.dtype).reshape(-1).copy_(src)
        return True


class HostKVCache:
    def __init__(self, mem_manager, bytes_budget: int, page_tokens: int = 64, disk_dir: Optional[str] = None,
                 disk_bytes: int = 0, staging_pages: int = 4, name: str = "rank0"):
        self.mm = mem_manager
        self.P = page_tokens
        self.device = mem_manager.kv_buffer.device
        self.cuda = self.device.type == "cuda"
        self.page_shape = (mem_manager.layer_num, page_tokens, *mem_manager.kv_row_shape())
        esz = torch.empty((), dtype=mem_manager.dtype).element_size()
        self.page_bytes = int(np.prod(self.page_shape)) * esz
        self.n_pages = max(1, int(bytes_budget) // self.page_bytes)
        from ..utils import host_memory as hm

        self.host_buffer = None
        if hm.huge_pages_wanted() or hm.numa_policy_wanted():
            # huge pages / NUMA placement asked for: own mapping, registered with CUDA, instead of torch's pinned pool
            self.host_buffer = hm.HostBuffer.create(
                self.n_pages * self.page_bytes, huge_pages=hm.huge_pages_wanted(), numa=hm.numa_policy_wanted(),
                device_index=self.device.index if self.cuda else None, register=self.cuda)
            self.pool = self.host_buffer.tensor(mem_manager.dtype, (self.n_pages, *self.page_shape))
            for note in self.host_buffer.notes:
                print(f"[host kv cache {name}] {note}", flush=True)
        else:
            self.pool = torch.empty((self.n_pages, *self.page_shape), dtype=mem_manager.dtype, pin_memory=self.cuda)
        self.index: "OrderedDict[bytes, int]" = OrderedDict()
        self.free = list(range(self.n_pages - 1, -1, -1))
        self.disk = None
        if disk_dir and disk_bytes > 0:
            self.disk = _DiskTier(os.path.join(disk_dir, f"llb_kv_{name}.bin"), int(disk_bytes) // self.page_bytes,
                                  self.page_shape, mem_manager.dtype)
        self.staging = [torch.empty(self.page_shape, dtype=mem_manager.dtype, device=self.device)
                        for _ in range(staging_pages)] if self.cuda else []
        self.stage_events = [None] * len(self.staging)
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._k = 0
        self.stats = {"offloaded_pages": 0, "loaded_pages": 0, "host_hits": 0, "disk_hits": 0, "evicted": 0}

    # ---- index ----
    def _take_page(self) -> int:
        if self.free:
            return self.free.pop()
        key, idx = self.index.popitem(last=False)
        self.stats["evicted"] += 1
        if self.disk is not None:
            self._wait_copies()
            self.disk.put(key, self.pool[idx])
        return idx

    def _wait_copies(self):
        if self.copy_stream is not None:
            self.copy_stream.synchronize()

    def match(self, keys: List[bytes], first_page: int) -> int:
        """Number of consecutive pages from `first_page` on held by this tier (host memory or disk)."""
        n = 0
        for k in keys[first_page:]:
            if k in self.index or (self.disk is not None and k in self.disk.index):
                n += 1
            else:
                break
        return n

    # ---- GPU -> host ----
    def offload(self, ids: np.ndarray, slots: np.ndarray) -> int:
        """Store the full pages of a finished sequence (`slots[i]` holds token i) that are not here yet."""
        keys = page_keys(ids, self.P)
        done = 0
        for p, k in enumerate(keys):
            if k in self.index:
                self.index.move_to_end(k)
                continue
            idx = self._take_page()
            s = torch.from_numpy(np.ascontiguousarray(slots[p * self.P:(p + 1) * self.P]))
            if self.cuda:
                j = self._k % len(self.staging)
                self._k += 1
                if self.stage_events[j] is not None:
                    torch.cuda.current_stream(self.device).wait_event(self.stage_events[j])
                self.mm.gather_pages(s, out=self.staging[j])
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(self.copy_stream):
                    self.copy_stream.wait_event(ready)
                    self.pool[idx].copy_(self.staging[j], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.copy_stream)
                self.stage_events[j] = ev
            else:
                self.mm.gather_pages(s, out=self.pool[idx])
            self.index[k] = idx
            done += 1
        self.stats["offloaded_pages"] += done
        return done

    # ---- host -> GPU ----
    def load(self, keys: List[bytes], first_page: int, n_pages: int, slots: torch.Tensor) -> None:
        """Copy pages [first_page, first_page + n_pages) into `slots` (n_pages * P pool slots)."""
        self._wait_copies()  # a page still on its way out must have landed before it is read back
        for i in range(n_pages):
            k = keys[first_page + i]
            s = slots[i * self.P:(i + 1) * self.P]
            idx = self.index.get(k)
            if idx is None:  # on disk: bring it back to host memory first
                idx = self._take_page()
                assert self.disk.get(k, self.pool[idx])
                self.index[k] = idx
                self.stats["disk_hits"] += 1
            else:
                self.index.move_to_end(k)
                self.stats["host_hits"] += 1
            if self.cuda:
                page = self.pool[idx].to(self.device, non_blocking=True)
                self.mm.scatter_pages(s, page)
            else:
                self.mm.scatter_pages(s, self.pool[idx])
        self.stats["loaded_pages"] += n_pages
