"""embed_cache process: serves `EmbedCache` over a zmq REP socket (pickled `(method, args)` calls), owns the
shared embedding arena.  `EmbedCacheClient` is the caller side used by the HTTP workers (alloc / release / payload
upload), the visual and audio servers (payload download, mark embedded) and LLM ranks (arena reads).
Reference: lightllm/server/embed_cache/manager.py, embed_cache_client.py.
"""
from __future__ import annotations

import pickle

import zmq

from ...utils.process_utils import set_proc_title, start_parent_check_thread
from ..core.objs.start_args import StartArgs
from .cache import EmbedArena, EmbedCache

METHODS = ("alloc", "release", "set_items_data", "get_items_data", "get_payload", "set_items_embed", "get_items_embed")


def arena_name(args) -> str:
    return f"{args.unique_server_name}_embed_arena"


def arena_rows(args, hidden: int) -> int:
    gb = float(getattr(args, "embed_cache_storage_size", 4) or 4)
    return max(1024, int(gb * (1 << 30)) // (hidden * 2))


def _id_range_source(args):
    if not (getattr(args, "config_server_host", None) and getattr(args, "config_server_port", None)):
        return None

    def take():
        import requests

        r = requests.get(f"http://{args.config_server_host}:{args.config_server_port}"
                         "/allocate_global_unique_multimodal_id_range", timeout=10)
        r.raise_for_status()
        j = r.json()
        return j["start_id"], j["end_id"]

    return take


def serve(cache: EmbedCache, sock, max_calls=None, stop=None):
    """Request loop; `stop` (threading.Event) ends it within 100 ms (the socket is only touched by this thread)."""
    n = 0
    while (max_calls is None or n < max_calls) and not (stop is not None and stop.is_set()):
        if not sock.poll(100):
            continue
        method, a = pickle.loads(sock.recv())
        n += 1
        try:
            if method not in METHODS:
                raise ValueError(f"unknown method {method}")
            res = ("ok", getattr(cache, method)(*a))
        except Exception as e:  # the caller gets the error, the server lives on
            res = ("err", repr(e))
        sock.send(pickle.dumps(res))


def start_cache_manager(args_dict: dict, hidden: int, pipe_writer):
    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::embed_cache")
    start_parent_check_thread()
    rows = arena_rows(args, hidden)
    arena = EmbedArena(arena_name(args), rows, hidden, create=True)
    cache = EmbedCache(args.cache_capacity, rows, _id_range_source(args))
    sock = zmq.Context(1).socket(zmq.REP)
    sock.bind(f"tcp://127.0.0.1:{args.cache_port}")
    pipe_writer.send("init ok")
    try:
        serve(cache, sock)
    finally:
        arena.close()


class EmbedCacheClient:
    def __init__(self, args, hidden: int = 0, open_arena: bool = False):
        self.sock = zmq.Context.instance().socket(zmq.REQ)
        self.sock.connect(f"tcp://127.0.0.1:{args.cache_port}")
        self.arena = EmbedArena(arena_name(args), arena_rows(args, hidden), hidden, create=False) if open_arena else None

    def _call(self, method, *a):
        self.sock.send(pickle.dumps((method, a)))
        st, res = pickle.loads(self.sock.recv())
        if st != "ok":
            raise RuntimeError(f"embed cache: {res}")
        return res

    def __getattr__(self, name):
        if name in METHODS:
            return lambda *a: self._call(name, *a)
        raise AttributeError(name)
