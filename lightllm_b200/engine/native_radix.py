"""Radix prefix cache backed by the C++ tree in ``csrc/runtime/runtime.cpp``.

Same interface and semantics as `radix_cache.RadixCache` (the Python tree is the executable
specification the C++ one is tested against); the model-rank hot path uses this one: matching a
4k-token prompt or inserting a finished request is a single native call.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import numpy as np

from ..ops._native import runtime

_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)


def _lib():
    lib = runtime()
    if not getattr(lib, "_radix_typed", False):
        lib.llb_radix_create.restype = ctypes.c_void_p
        lib.llb_radix_destroy.argtypes = [ctypes.c_void_p]
        lib.llb_radix_total_tokens.restype = ctypes.c_int64
        lib.llb_radix_total_tokens.argtypes = [ctypes.c_void_p]
        lib.llb_radix_refed_tokens.restype = ctypes.c_int64
        lib.llb_radix_refed_tokens.argtypes = [ctypes.c_void_p]
        lib.llb_radix_insert.restype = ctypes.c_int64
        lib.llb_radix_insert.argtypes = [ctypes.c_void_p, _i64p, _i32p, ctypes.c_int64]
        lib.llb_radix_match.restype = ctypes.c_int64
        lib.llb_radix_match.argtypes = [ctypes.c_void_p, _i64p, ctypes.c_int64, ctypes.c_int32, _i32p,
                                        ctypes.POINTER(ctypes.c_void_p)]
        lib.llb_radix_add_ref.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.llb_radix_dec_ref.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.llb_radix_dec_ref.restype = ctypes.c_int32
        lib.llb_radix_evict.restype = ctypes.c_int64
        lib.llb_radix_evict.argtypes = [ctypes.c_void_p, ctypes.c_int64, _i32p, ctypes.c_int64]
        lib.llb_radix_merge.restype = ctypes.c_int64
        lib.llb_radix_merge.argtypes = [ctypes.c_void_p]
        lib.llb_radix_node_count.restype = ctypes.c_int64
        lib.llb_radix_node_count.argtypes = [ctypes.c_void_p]
        lib._radix_typed = True
    return lib


class NativeRadixCache:
    def __init__(self, unique_name: str = "radix", total_token_num: int = 0, rank_in_node: int = 0, mem_manager=None,
                 shared_counters=None):
        self._lib = _lib()
        self._h = ctypes.c_void_p(self._lib.llb_radix_create())
        self.mem_manager = mem_manager
        self._shared = shared_counters

    def __del__(self):
        try:
            if self._h:
                self._lib.llb_radix_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def _publish(self):
        if self._shared is not None:
            self._shared.set(self.get_refed_tokens_num(), self.get_tree_total_tokens_num())

    def get_refed_tokens_num(self) -> int:
        return int(self._lib.llb_radix_refed_tokens(self._h))

    def get_tree_total_tokens_num(self) -> int:
        return int(self._lib.llb_radix_total_tokens(self._h))

    def unreferenced_tokens_num(self) -> int:
        return self.get_tree_total_tokens_num() - self.get_refed_tokens_num()

    def node_count(self) -> int:
        return int(self._lib.llb_radix_node_count(self._h))

    def insert(self, key, value) -> int:
        key = np.ascontiguousarray(key, dtype=np.int64)
        value = np.ascontiguousarray(value, dtype=np.int32)
        assert key.shape[0] == value.shape[0]
        n = self._lib.llb_radix_insert(self._h, key.ctypes.data_as(_i64p), value.ctypes.data_as(_i32p), key.shape[0])
        self._publish()
        return int(n)

    def match_prefix(self, key, update_refs: bool = False):
        key = np.ascontiguousarray(key, dtype=np.int64)
        n = key.shape[0]
        if n == 0:
            return None, 0, None
        out = np.empty(n, dtype=np.int32)
        node = ctypes.c_void_p()
        m = int(self._lib.llb_radix_match(self._h, key.ctypes.data_as(_i64p), n, 1 if update_refs else 0,
                                          out.ctypes.data_as(_i32p), ctypes.byref(node)))
        if m == 0:
            return None, 0, None
        if update_refs:
            self._publish()
        return node.value, m, out[:m]

    def add_node_ref_counter(self, node):
        if node:
            self._lib.llb_radix_add_ref(self._h, ctypes.c_void_p(node))
            self._publish()

    def dec_node_ref_counter(self, node):
        if node:
            rc = self._lib.llb_radix_dec_ref(self._h, ctypes.c_void_p(node))
            assert rc == 0, "radix reference count underflow"
            self._publish()

    def evict(self, need_remove_tokens: int, evict_callback: Callable[[np.ndarray], None]) -> int:
        if need_remove_tokens <= 0:
            return 0
        cap = max(self.unreferenced_tokens_num(), 1)
        out = np.empty(cap, dtype=np.int32)
        n = int(self._lib.llb_radix_evict(self._h, need_remove_tokens, out.ctypes.data_as(_i32p), cap))
        if n:
            evict_callback(out[:n])
        self._publish()
        return n

    def free_radix_cache_to_get_enough_token(self, need_token_num: int):
        if self.mem_manager is None:
            return
        free = self.mem_manager.can_use_mem_size
        if need_token_num > free:
            self.evict(need_token_num - free, lambda v: self.mem_manager.free(v))

    def publish(self, key, slots) -> int:
        """Hand externally filled slots (KV that arrived from another node or cache tier) to the tree under
        `key`; copies of positions the tree already had are returned to the pool.  Returns that count."""
        v = np.asarray(slots.cpu() if hasattr(slots, "cpu") else slots, dtype=np.int32)
        k = np.asarray(key.cpu() if hasattr(key, "cpu") else key, dtype=np.int64)
        present = self.insert(k, v)
        if present and self.mem_manager is not None:
            self.mem_manager.free(v[:present])
        return present

    def clear_tree_nodes(self):
        self.evict(self.get_tree_total_tokens_num(), lambda v: self.mem_manager.free(v) if self.mem_manager else None)

    def merge_unreferenced_nodes(self) -> int:
        """Merges chains of unreferenced single-child nodes; returns how many nodes went away."""
        return int(self._lib.llb_radix_merge(self._h))
