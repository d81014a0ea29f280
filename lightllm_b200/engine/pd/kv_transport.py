"""KV transfer between a prefill rank and a decode rank (PD disaggregation).

One link = a control connection (length-prefixed JSON headers over TCP, opened with an HMAC challenge on a
per-deployment secret) + a 2-rank process group for the payload (NCCL send/recv between GPUs, gloo for CPU pools).  The payload unit is a staged page
`[L, page_tokens, rows...]` gathered from the sender's token-granular pool; the receiver lands it in one of
`page_num` staging pages and the decode rank's inference loop scatters it into freshly allocated pool slots
(`drain`).  When the last page of a request is in, the slots are published to the decode node's prefix
cache under the request's prompt token ids, so the follow-up request (prompt + first token) finds the whole
prompt cached and starts decoding at once; no separate "KV-ready" request path exists.

A header always travels on the control connection before its payload is posted, so a device-side receive
is only ever enqueued when the matching send is already on its way.
Both ranks of a link must hold the same KV head shard (equal tp on the P and D node).

Reference: lightllm/server/router/model_infer/mode_backend/pd/nccl_kv_transporter.py,
prefill_node_impl/prefill_impl.py:50-92, decode_node_impl/decode_impl.py.
"""
from __future__ import annotations

import datetime
import hashlib
import json
import os
import queue
import threading
import time
from dataclasses import asdict, dataclass, field
from multiprocessing.connection import Client, Connection, Listener
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

TASK_TIMEOUT_S = 182.0
CONNECT_TIMEOUT_S = 8.0
LINK_RETRY_S = 10.0      # a peer that failed is not tried again for this long: queued requests fail at once


def auth_key() -> bytes:
    """Secret of the control connections.  Every node of one deployment must be started with the same
    `--pd_kv_auth_key` (or LLB_PD_KV_AUTHKEY); without one the key is derived from the pd_master address, which
    keeps strangers of another deployment out but is no protection against someone who knows that address."""
    k = os.environ.get("LLB_PD_KV_AUTHKEY")
    if k:
        return hashlib.sha256(k.encode()).digest()
    seed = os.environ.get("LLB_PD_MASTER_ADDR", "standalone")
    return hashlib.sha256(("llb-pd-kv:" + seed).encode()).digest()


@dataclass
class PageHeader:
    group_req_id: int
    page_index: int
    num_tokens: int
    last: bool
    token_ids: Optional[List[int]] = None  # on the last page: the request's prompt ids (prefix-cache key)
    first_token: Optional[tuple] = None
    created: float = field(default_factory=time.time)

    def encode(self) -> bytes:
        return json.dumps(asdict(self), separators=(",", ":")).encode()

    @staticmethod
    def decode(raw: bytes) -> Optional["PageHeader"]:
        d = json.loads(raw.decode())
        if d is None:
            return None
        ft = d.get("first_token")
        ids = d.get("token_ids")
        return PageHeader(int(d["group_req_id"]), int(d["page_index"]), int(d["num_tokens"]), bool(d["last"]),
                          [int(x) for x in ids] if ids is not None else None,
                          (int(ft[0]), float(ft[1])) if ft is not None else None, float(d.get("created", 0.0)))


def _connect(peer: Tuple[str, int], timeout_s: float) -> Connection:
    """Client(peer) with a limit on how long an unreachable peer may take."""
    box: dict = {}

    def run():
        try:
            box["conn"] = Client(peer, authkey=auth_key())
        except BaseException as e:  # noqa: BLE001
            box["err"] = e

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(timeout_s)
    if "conn" in box:
        return box["conn"]
    raise ConnectionError(f"KV link to {peer}: {box.get('err', 'no answer within %.0f s' % timeout_s)}")


def _make_group(store, rank: int, cuda: bool, timeout_s: float):
    td = datetime.timedelta(seconds=timeout_s)
    if cuda:
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = td
        return dist.ProcessGroupNCCL(store, rank, 2, opts)
    return dist.ProcessGroupGloo(store, rank, 2, td)


class _Link:
    def __init__(self, conn: Connection, pg, rank: int):
        self.conn, self.pg, self.rank = conn, pg, rank
        self.lock = threading.Lock()


class KVSender:
    """Prefill-rank side.  `send_request` streams one finished prefill to a decode rank and returns when it is
    out; `submit` queues the same work for a worker thread (the inference loop keeps running and collects the
    outcomes with `poll_done`).  The caller must keep the slots alive until the outcome is in."""

    def __init__(self, mem_manager, page_tokens: int = 1024, timeout_s: float = TASK_TIMEOUT_S,
                 connect_timeout_s: float = CONNECT_TIMEOUT_S):
        self.mm, self.page_tokens, self.timeout_s = mem_manager, page_tokens, timeout_s
        self.connect_timeout_s = connect_timeout_s
        self.links: Dict[Tuple[str, int], _Link] = {}
        self.broken: Dict[Tuple[str, int], float] = {}
        self.cuda = mem_manager.kv_buffer.is_cuda
        self.stage = torch.empty((mem_manager.layer_num, page_tokens, *mem_manager.kv_row_shape()),
                                 dtype=mem_manager.dtype, device=mem_manager.kv_buffer.device)
        self.stream = torch.cuda.Stream() if self.cuda else None
        self._tasks: "queue.Queue" = queue.Queue()
        self._done: "queue.Queue" = queue.Queue()
        self._worker: Optional[threading.Thread] = None

    def _link(self, peer: Tuple[str, int]) -> _Link:
        lk = self.links.get(peer)
        if lk is None:
            since = self.broken.get(peer)
            if since is not None and time.time() - since < LINK_RETRY_S:
                raise ConnectionError(f"KV link to {peer} failed {time.time() - since:.1f} s ago")
            conn = _connect(peer, self.connect_timeout_s)
            if not conn.poll(self.connect_timeout_s):
                conn.close()
                raise ConnectionError(f"KV link to {peer}: no rendezvous port within {self.connect_timeout_s:.0f} s")
            store_port = int(json.loads(conn.recv_bytes().decode()))  # the receiver hosts the link's rendezvous store
            store = dist.TCPStore(peer[0], store_port, 2, False,
                                  timeout=datetime.timedelta(seconds=max(self.connect_timeout_s, 1.0)))
            lk = self.links[peer] = _Link(conn, _make_group(store, 0, self.cuda, self.timeout_s), 0)
            self.broken.pop(peer, None)
        return lk

    def send_request(self, peer: Tuple[str, int], group_req_id: int, token_ids: List[int], slots: torch.Tensor,
                     first_token: Optional[tuple] = None) -> int:
        """Gather `slots` page by page and send them; returns the number of pages."""
        try:
            return self._send(peer, group_req_id, token_ids, slots, first_token)
        except BaseException:
            lk = self.links.pop(peer, None)   # the link's state is unknown after a failure: start over next time
            self.broken[peer] = time.time()
            if lk is not None:
                try:
                    lk.conn.close()
                except Exception:
                    pass
            raise

    def _send(self, peer, group_req_id, token_ids, slots, first_token) -> int:
        lk = self._link(peer)
        n = int(slots.shape[0])
        pages = max(1, (n + self.page_tokens - 1) // self.page_tokens)
        with lk.lock:
            for p in range(pages):
                s, e = p * self.page_tokens, min(n, (p + 1) * self.page_tokens)
                last = p == pages - 1
                hdr = PageHeader(group_req_id, p, e - s, last, [int(t) for t in token_ids[:n]] if last else None,
                                 first_token if last else None).encode()
                if self.cuda:
                    if threading.current_thread() is not self._worker:
                        self.stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(self.stream):
                        self.mm.gather_pages(slots[s:e], out=self.stage[:, : e - s])
                        lk.conn.send_bytes(hdr)
                        lk.pg.send([self.stage], 1, 0).wait()
                    self.stream.synchronize()
                else:
                    self.mm.gather_pages(slots[s:e], out=self.stage[:, : e - s])
                    lk.conn.send_bytes(hdr)
                    lk.pg.send([self.stage], 1, 0).wait()
        return pages

    # ---- asynchronous use ----
    def submit(self, peer: Tuple[str, int], group_req_id: int, token_ids: List[int], slots: torch.Tensor,
               first_token: Optional[tuple] = None, tag=None):
        """Queue one request.  `slots` is copied; the KV rows themselves are read by the worker, so the pool slots
        must stay allocated until `poll_done` reports `tag` (default: the group request id)."""
        if self._worker is None:
            self._worker = threading.Thread(target=self._work, daemon=True)
            self._worker.start()
        if self.cuda:
            # the KV rows were written on the caller's stream: the worker's gathers must come after them
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
        else:
            ev = None
        self._tasks.put((peer, group_req_id, list(token_ids), slots.clone(), first_token,
                         group_req_id if tag is None else tag, ev))

    def _work(self):
        if self.cuda:
            torch.cuda.set_device(self.mm.kv_buffer.device)
        while True:
            task = self._tasks.get()
            if task is None:
                return
            peer, gid, ids, slots, first, tag, ev = task
            try:
                if ev is not None:
                    self.stream.wait_event(ev)
                self.send_request(peer, gid, ids, slots, first)
                self._done.put((tag, True, None))
            except BaseException as e:  # noqa: BLE001
                self._done.put((tag, False, f"{type(e).__name__}: {e}"))

    def poll_done(self) -> List[Tuple[object, bool, Optional[str]]]:
        out = []
        while True:
            try:
                out.append(self._done.get_nowait())
            except queue.Empty:
                return out

    def close(self):
        if self._worker is not None:
            self._tasks.put(None)
        for lk in self.links.values():
            try:
                lk.conn.send_bytes(b"null")
                lk.conn.close()
            except Exception:
                pass
        self.links.clear()


class KVReceiver:
    """Decode-rank side: a listener thread accepts links, one thread per link lands pages in the staging ring;
    `drain()` (called by the inference loop between steps) moves landed pages into the pool."""

    def __init__(self, mem_manager, host: str, port: int, page_tokens: int = 1024, page_num: int = 16,
                 timeout_s: float = TASK_TIMEOUT_S):
        self.mm, self.page_tokens, self.timeout_s = mem_manager, page_tokens, timeout_s
        self.cuda = mem_manager.kv_buffer.is_cuda
        dev = mem_manager.kv_buffer.device
        self.pages = [torch.empty((mem_manager.layer_num, page_tokens, *mem_manager.kv_row_shape()),
                                  dtype=mem_manager.dtype, device=dev) for _ in range(page_num)]
        self.free_pages: "queue.Queue[int]" = queue.Queue()
        for i in range(page_num):
            self.free_pages.put(i)
        self.landed: "queue.Queue[Tuple[PageHeader, int]]" = queue.Queue()
        self.partial: Dict[int, Optional[List[torch.Tensor]]] = {}  # gid -> slot tensors so far (None: failed)
        self.staged: Dict[int, Tuple[PageHeader, int]] = {}  # key gid * 65536 + page -> landed, not yet in the pool
        self.host = host
        self.listener = Listener((host, port), authkey=auth_key())
        self.port = self.listener.address[1]
        self.stream = torch.cuda.Stream() if self.cuda else None
        self._stop = False
        self._threads: List[threading.Thread] = []
        t = threading.Thread(target=self._accept_loop, daemon=True)
        t.start()
        self._threads.append(t)

    def _accept_loop(self):
        while not self._stop:
            try:
                conn = self.listener.accept()
            except (OSError, EOFError) as e:
                if self._stop or getattr(e, "errno", None) in (9, 22):   # listener closed
                    return
                continue
            except Exception:   # a peer that failed the challenge: keep listening
                continue
            t = threading.Thread(target=self._link_loop, args=(conn,), daemon=True)
            t.start()
            self._threads.append(t)

    def _link_loop(self, conn: Connection):
        if self.cuda:
            torch.cuda.set_device(self.mm.kv_buffer.device)
        store = dist.TCPStore(self.host, 0, 2, True, timeout=datetime.timedelta(seconds=60), wait_for_workers=False)
        conn.send_bytes(json.dumps(store.port).encode())
        pg = _make_group(store, 1, self.cuda, self.timeout_s)
        while not self._stop:
            try:
                hdr = PageHeader.decode(conn.recv_bytes(1 << 26))
            except (EOFError, OSError, ValueError, KeyError, TypeError):
                return
            if hdr is None or not (0 < hdr.num_tokens <= self.page_tokens):
                return
            idx = self.free_pages.get()
            page = self.pages[idx]
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    pg.recv([page], 0, 0).wait()
                self.stream.synchronize()
            else:
                pg.recv([page], 0, 0).wait()
            self.landed.put((hdr, idx))

    def has_landed(self) -> bool:
        return not self.landed.empty() or bool(self.staged)

    def drain(self, prefix_cache=None, agree=None) -> List[Tuple[int, bool, Optional[tuple]]]:
        """Scatter landed pages into the pool.  Returns `(group_req_id, ok, first_token)` for every request that
        completed (ok False: the pool could not hold it).

        With tensor parallelism every rank of the decode node runs its own receiver, and their pools and prefix
        trees must change in the same order: `agree(keys) -> keys` returns the page keys that have landed on
        all ranks (a collective the caller supplies); only those are processed, in sorted order, the rest wait
        in their staging pages."""
        while True:
            try:
                hdr, idx = self.landed.get_nowait()
            except queue.Empty:
                break
            self.staged[hdr.group_req_id * 65536 + hdr.page_index] = (hdr, idx)
        keys = sorted(self.staged)
        if agree is not None:
            keys = sorted(agree(keys))
        done = []
        for key in keys:
            hdr, idx = self.staged.pop(key)
            slots = None
            try:
                failed = self.partial.get(hdr.group_req_id, []) is None
                if not failed:
                    if self.mm.can_use_mem_size < hdr.num_tokens and prefix_cache is not None:
                        prefix_cache.free_radix_cache_to_get_enough_token(hdr.num_tokens)
                    if self.mm.can_use_mem_size >= hdr.num_tokens:
                        # alloc() hands out a view of a small ring of host buffers that later allocations
                        # (further pages, decode steps between two drains) reuse: keep a copy
                        slots = self.mm.alloc(hdr.num_tokens).clone()
                        self.mm.scatter_pages(slots, self.pages[idx][:, : hdr.num_tokens])
                        if self.cuda:
                            torch.cuda.current_stream().synchronize()
                    else:
                        failed = True
            finally:
                self.free_pages.put(idx)
            if failed:
                for s in self.partial.get(hdr.group_req_id) or []:
                    self.mm.free(s)
                self.partial[hdr.group_req_id] = None  # later pages of a failed request are dropped
                if hdr.last:
                    self.partial.pop(hdr.group_req_id, None)
                    done.append((hdr.group_req_id, False, None))
                continue
            self.partial.setdefault(hdr.group_req_id, []).append(slots)
            if hdr.last:
                all_slots = torch.cat(self.partial.pop(hdr.group_req_id))
                if prefix_cache is not None:
                    prefix_cache.publish(torch.tensor(hdr.token_ids, dtype=torch.int64), all_slots)
                else:
                    self.mm.free(all_slots)
                done.append((hdr.group_req_id, True, hdr.first_token))
        return done

    def close(self):
        self._stop = True
        try:
            self.listener.close()
        except Exception:
            pass
