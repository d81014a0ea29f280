"""Vision encoders as a service of their own: `--run_mode visual_only` runs a vision tower that registers at the
config server; language-model servers started with `--visual_use_proxy_mode` keep no tower and send their
pictures to one of the registered encoders.

An encoder listens on a ZeroMQ ROUTER socket (`--visual_rpyc_port`).  A request is one pickled
`(request id, [(item, payload bytes), ...])`; the answer carries the embeddings inline, one tensor per item, so
the two sides need no shared file system.  Every message carries an HMAC-SHA256 signature (`LLB_VIT_AUTHKEY`, else
a key derived from the config server's address) that is checked before the body is unpickled.  With `--afs_image_embed_dir` (a directory that all servers see) the
encoders also keep every embedding there under the picture's content hash, at most `--afs_embed_capacity` files
(least recently used first out), and both sides look there before they compute or ask: a picture embedded once
is not sent again, whichever server meets it next.

The proxy side replaces the tower pass of `VisualManager` only: cache records, the arena and the hand-over to the
router are unchanged.  Encoders come and go: the proxy polls the config server's list, sends each batch to one
encoder and retries once on another when no answer comes within `LLB_REMOTE_VIT_TIMEOUT_S` (default 600 s).

Reference: lightllm/server/visualserver/proxy_manager.py, visual_only_manager.py, objs.py (VIT_Obj),
lightllm/server/embed_cache/afs_utils.py (its ready marks live in redis; here the file itself is the mark).
"""
from __future__ import annotations

import base64
import itertools
import os
import pickle
import random
import tempfile
import threading
import time
import traceback
import uuid
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import zmq

from ...utils.process_utils import set_proc_title, start_parent_check_thread
from ...utils.log_utils import init_logger
from ...utils.signed_msg import derive_key, seal, unseal

logger = init_logger(__name__)
from ..core.objs.start_args import StartArgs
from .manager import VisualManager, build_vision_tower, open_req_table


def auth_key(args=None) -> bytes:
    """Key of the message signatures between servers and encoders: `LLB_VIT_AUTHKEY` (the same on every machine of
    a deployment) or, without it, a key derived from the config server's address."""
    return derive_key("LLB_VIT_AUTHKEY", f"{getattr(args, 'config_server_host', None)}:"
                                         f"{getattr(args, 'config_server_port', None)}")


def remote_timeout_s() -> float:
    return float(os.environ.get("LLB_REMOTE_VIT_TIMEOUT_S", "600"))


@dataclass
class VitNode:
    node_id: int
    host_ip: str
    port: int

    @property
    def host_ip_port(self) -> str:
        return f"{self.host_ip}:{self.port}"


# ------------------------------------------------------------------ shared directory of embeddings
class SharedEmbedDir:
    """Embeddings by content hash in a directory every server can reach.  A file appears under its final name only
    when complete (written aside, then renamed), so its presence is the "ready" mark; reading one refreshes its
    time stamp and the oldest files go when there are more than `capacity`."""

    RESCAN_EVERY = 4096   # stores between two full counts (other writers share the directory)

    def __init__(self, root: str, capacity: int = 250000):
        self.root, self.capacity = root, max(1, int(capacity))
        os.makedirs(root, exist_ok=True)
        self._count = len(self._files())      # files believed to be there; exact after every scan
        self._since_scan = 0

    def _path(self, md5: str) -> str:
        return os.path.join(self.root, md5[:2], md5 + ".pt")

    def has(self, md5: str) -> bool:
        return bool(md5) and os.path.exists(self._path(md5))

    def load(self, md5: str) -> Optional[torch.Tensor]:
        if not md5:
            return None
        p = self._path(md5)
        try:
            t = torch.load(p, map_location="cpu", weights_only=True)
            os.utime(p, None)
            return t
        except Exception:  # noqa: BLE001  (missing, torn or foreign file: a miss)
            return None

    def store(self, md5: str, emb: torch.Tensor):
        if not md5:
            return
        p = self._path(md5)
        fresh = not os.path.exists(p)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=os.path.dirname(p), suffix=".part")
        try:
            with os.fdopen(fd, "wb") as f:
                torch.save(emb.detach().cpu().contiguous(), f)
            os.replace(tmp, p)
        except BaseException:
            try:
                os.unlink(tmp)
            except OSError:
                pass
            raise
        self._count += int(fresh)
        self._since_scan += 1
        if self._count > self.capacity or self._since_scan >= self.RESCAN_EVERY:
            self.sweep()

    def _files(self):
        files = []
        try:
            subs = os.listdir(self.root)
        except OSError:
            return files
        for sub in subs:
            d = os.path.join(self.root, sub)
            if not os.path.isdir(d):
                continue
            for name in os.listdir(d):
                if name.endswith(".pt"):
                    try:
                        files.append((os.path.getmtime(os.path.join(d, name)), os.path.join(d, name)))
                    except OSError:
                        pass
        return files

    def sweep(self):
        """Counts the files and removes the least recently used ones above the capacity (a little more than
        needed, so that a full directory is not scanned on every store)."""
        files = self._files()
        self._since_scan = 0
        extra = len(files) - self.capacity
        if extra > 0:
            extra = min(len(files), extra + self.capacity // 50)
            for _, p in sorted(files)[:extra]:
                try:
                    os.unlink(p)
                except OSError:
                    pass
            self._count = len(files) - extra
        else:
            self._count = len(files)


def shared_dir_of(args) -> Optional[SharedEmbedDir]:
    d = getattr(args, "afs_image_embed_dir", None)
    return SharedEmbedDir(d, getattr(args, "afs_embed_capacity", 250000) or 250000) if d else None


# ------------------------------------------------------------------ encoder side
class VisualOnlyServer:
    """Serves embedding requests with a local tower."""

    def __init__(self, tower, sock, shared: Optional[SharedEmbedDir] = None, infer_batch_size: int = 8,
                 key: Optional[bytes] = None):
        self.tower, self.sock, self.shared = tower, sock, shared
        self.key = key or auth_key()
        self.infer_batch_size = max(1, int(infer_batch_size or 1))
        self.served = 0          # tower passes' pictures (not counting shared-directory hits)

    def encode(self, pairs: List[Tuple[dict, bytes]]) -> List[torch.Tensor]:
        out: List[Optional[torch.Tensor]] = [None] * len(pairs)
        first: Dict[str, int] = {}
        todo = []
        for i, (item, _) in enumerate(pairs):
            key = item.get("md5") or f"#{i}"
            if key in first:
                continue
            first[key] = i
            hit = self.shared.load(item.get("md5")) if self.shared is not None else None
            if hit is not None and hit.shape[0] == item["token_num"]:
                out[i] = hit
            else:
                todo.append(i)
        for s in range(0, len(todo), self.infer_batch_size):
            idx = todo[s:s + self.infer_batch_size]
            embs = self.tower.encode_images([pairs[i][1] for i in idx], items=[pairs[i][0] for i in idx])
            for i, e in zip(idx, embs):
                item = pairs[i][0]
                if e.shape[0] != item["token_num"]:
                    raise ValueError(f"image gives {e.shape[0]} tokens, the prompt reserved {item['token_num']}")
                out[i] = e.detach().to("cpu")
                self.served += 1
                if self.shared is not None:
                    self.shared.store(item.get("md5"), out[i])
        for i, (item, _) in enumerate(pairs):       # repeats of one picture inside a request
            if out[i] is None:
                out[i] = out[first[item.get("md5") or f"#{i}"]]
        return out

    def serve_one(self, timeout_ms: Optional[int] = None) -> bool:
        if timeout_ms is not None and not self.sock.poll(timeout_ms):
            return False
        ident, *frames = self.sock.recv_multipart()
        rid = None
        try:
            rid, pairs = unseal(self.key, frames)
            reply = (rid, "ok", self.encode(pairs))
        except PermissionError as e:
            logger.warning(f"dropped a request: {e}")
            return True               # no answer to a stranger
        except Exception as e:  # noqa: BLE001
            traceback.print_exc()
            reply = (rid, "error", f"{type(e).__name__}: {e}")
        self.sock.send_multipart([ident] + seal(self.key, reply))
        return True

    def loop(self, stop: Optional[threading.Event] = None):
        while stop is None or not stop.is_set():
            self.serve_one(200)


def keep_registered(node: VitNode, host: str, port: int, stop: Optional[threading.Event] = None, beat_s: float = 10.0):
    """Holds a websocket to the config server's `/visual_register` (the entry lives as long as the socket does) and
    opens it again when it breaks.  Runs until `stop` is set."""
    import asyncio

    import websockets

    async def run():
        while stop is None or not stop.is_set():
            try:
                async with websockets.connect(f"ws://{host}:{port}/visual_register", max_size=None) as ws:
                    await ws.send(pickle.dumps(node))
                    last = 0.0
                    while stop is None or not stop.is_set():
                        if time.time() - last >= beat_s:
                            await ws.send("beat")
                            last = time.time()
                        await asyncio.sleep(0.2)
            except Exception as e:  # noqa: BLE001
                logger.warning(f"config server {host}:{port} not reachable ({type(e).__name__}); retrying")
                await asyncio.sleep(2.0)

    asyncio.run(run())


def address_towards(host: str, port: int) -> str:
    """This machine's address on the route to `host` (what the other servers can reach an encoder under when it
    listens on all interfaces); 127.0.0.1 when no route is known."""
    import socket

    s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
    try:
        s.connect((host, port))           # no packet is sent: the kernel only picks the source address
        return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"
    finally:
        s.close()


def start_visual_only_process(args_dict: dict, pipe_writer=None):
    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::visual_only_server")
    start_parent_check_thread()
    try:
        assert args.visual_rpyc_port, "--run_mode visual_only needs --visual_rpyc_port (the port encoders are asked on)"
        assert args.config_server_host and args.config_server_port, \
            "--run_mode visual_only needs --config_server_host / --config_server_port to be found by the servers"
        dev_index = (args.visual_gpu_ids or [0])[0] if torch.cuda.is_available() else None
        device = torch.device("cuda", dev_index) if dev_index is not None else torch.device("cpu")
        tower = build_vision_tower(args, device, torch.bfloat16 if device.type == "cuda" else torch.float32)
        sock = zmq.Context(2).socket(zmq.ROUTER)
        sock.bind(f"tcp://{args.host if args.host not in (None, '') else '0.0.0.0'}:{args.visual_rpyc_port}")
        server = VisualOnlyServer(tower, sock, shared_dir_of(args), args.visual_infer_batch_size or 8, key=auth_key(args))
        node = VitNode(getattr(args, "visual_node_id", None) or uuid.uuid4().int & ((1 << 62) - 1),
                       args.host if args.host not in (None, "", "0.0.0.0") else
                       address_towards(args.config_server_host, int(args.config_server_port)), int(args.visual_rpyc_port))
        threading.Thread(target=keep_registered, args=(node, args.config_server_host, int(args.config_server_port)),
                         daemon=True).start()
    except Exception:
        if pipe_writer is not None:
            pipe_writer.send(("init failed", traceback.format_exc()))
        raise
    if pipe_writer is not None:
        pipe_writer.send("init ok")
    server.loop()


# ------------------------------------------------------------------ proxy side
class RemoteEncoders:
    """The encoders known to the config server, one DEALER socket each (used by one thread)."""

    def __init__(self, host: Optional[str], port: Optional[int], fetch=None):
        self.host, self.port = host, port
        self._fetch = fetch or self._http_fetch
        self.nodes: Dict[int, VitNode] = {}
        self.socks: Dict[int, "zmq.Socket"] = {}
        self.ctx = zmq.Context.instance()
        self._last, self._rr = 0.0, itertools.count()

    def _http_fetch(self) -> List[VitNode]:
        import requests

        r = requests.get(f"http://{self.host}:{self.port}/registered_visual_objects", timeout=10)
        r.raise_for_status()
        return list(pickle.loads(base64.b64decode(r.json()["data"])))

    def refresh(self, force: bool = False):
        """Every 10 s while no encoder is known, every 30 s otherwise (or at once with `force`)."""
        now = time.time()
        if not force and now - self._last < (30.0 if self.nodes else 10.0):
            return
        self._last = now
        try:
            listed = {n.node_id: n for n in self._fetch()}
        except Exception as e:  # noqa: BLE001
            logger.warning(f"cannot list the encoders ({type(e).__name__}: {e})")
            return
        for nid in list(self.nodes):
            if nid not in listed or listed[nid].host_ip_port != self.nodes[nid].host_ip_port:
                self.drop(nid)
        for nid, n in listed.items():
            if nid not in self.nodes:
                s = self.ctx.socket(zmq.DEALER)
                s.setsockopt(zmq.LINGER, 0)
                s.connect(f"tcp://{n.host_ip}:{n.port}")
                self.nodes[nid], self.socks[nid] = n, s

    def drop(self, nid: int):
        self.nodes.pop(nid, None)
        s = self.socks.pop(nid, None)
        if s is not None:
            s.close(0)

    def pick(self, avoid=()) -> Optional[int]:
        ids = [i for i in self.nodes if i not in avoid]
        if not ids:
            return None
        return ids[(next(self._rr) + random.randrange(len(ids))) % len(ids)]

    def close(self):
        for nid in list(self.socks):
            self.drop(nid)


class ProxyVisualManager(VisualManager):
    """`VisualManager` whose tower pass happens on a registered encoder."""

    LOOK_EVERY_S = 5.0      # while waiting for an answer: how often to ask whether the encoder is still registered

    def __init__(self, args, cache=None, send_next=None, recv=None, infer_batch_size: int = 8, try_recv=None,
                 send_batch_size: int = 1, encoders: Optional[RemoteEncoders] = None,
                 shared: Optional[SharedEmbedDir] = None, timeout_s: Optional[float] = None,
                 key: Optional[bytes] = None):
        super().__init__(args, None, cache, send_next, recv, infer_batch_size, try_recv, send_batch_size)
        self.encoders = encoders or RemoteEncoders(getattr(args, "config_server_host", None),
                                                   getattr(args, "config_server_port", None))
        self.shared = shared if shared is not None else shared_dir_of(args)
        self.timeout_s = remote_timeout_s() if timeout_s is None else timeout_s
        self.key = key or auth_key(args)
        self._rid = itertools.count(1)

    def _publish(self, item: dict, emb: torch.Tensor):
        assert emb.shape[0] == item["token_num"], \
            f"image gives {emb.shape[0]} tokens, the prompt reserved {item['token_num']}"
        self.cache.arena.write(item["start_index_in_embed_cache"], emb)

    def _ask(self, nid: int, pairs) -> List[torch.Tensor]:
        sock = self.encoders.socks[nid]
        rid = next(self._rid)
        sock.send_multipart(seal(self.key, (rid, pairs)))
        where = self.encoders.nodes[nid].host_ip_port
        deadline = time.time() + self.timeout_s
        next_look = time.time() + self.LOOK_EVERY_S
        while True:
            left = deadline - time.time()
            if left <= 0 or not sock.poll(int(min(left, 1.0) * 1000) + 1):
                if left <= 0:
                    raise TimeoutError(f"encoder {where}: no answer in {self.timeout_s:.0f} s")
                if time.time() >= next_look:      # an encoder that died has left the config server's list by now
                    next_look = time.time() + self.LOOK_EVERY_S
                    self.encoders.refresh(force=True)
                    if nid not in self.encoders.nodes:
                        raise ConnectionError(f"encoder {where} is no longer registered")
                continue
            try:
                got, status, body = unseal(self.key, sock.recv_multipart())
            except PermissionError:
                continue
            if got != rid:
                continue              # a late answer to a request that was given up
            if status != "ok":
                raise RuntimeError(f"encoder {self.encoders.nodes[nid].host_ip_port}: {body}")
            return body

    def embed(self, images: List[dict]):
        uniq = {i["uuid"]: i for i in images}
        todo = []
        for it in uniq.values():
            hit = self.shared.load(it.get("md5")) if self.shared is not None else None
            if hit is not None and hit.shape[0] == it["token_num"]:
                self._publish(it, hit)
                self.cache.set_items_embed([it["uuid"]])
            else:
                todo.append(it)
        if not todo:
            return
        self.encoders.refresh(force=not self.encoders.nodes)
        for s in range(0, len(todo), self.infer_batch_size):
            chunk = todo[s:s + self.infer_batch_size]
            pairs = [({k: v for k, v in it.items()}, self.cache.get_payload(it["uuid"])) for it in chunk]
            tried, embs, err = [], None, None
            for _ in range(2):
                nid = self.encoders.pick(avoid=tried)
                if nid is None:
                    break
                tried.append(nid)
                try:
                    embs = self._ask(nid, pairs)
                    break
                except Exception as e:  # noqa: BLE001
                    err = e
                    logger.warning(f"{e}")
                    if nid in self.encoders.nodes:
                        self.encoders.drop(nid)  # listed again at the next refresh if it is still registered
                    self.encoders._last = 0.0
            if embs is None:
                raise RuntimeError(f"no vision encoder answered ({err or 'none is registered at the config server'})")
            for it, e in zip(chunk, embs):
                self._publish(it, e)
            self.cache.set_items_embed([it["uuid"] for it in chunk])

    def handle_many(self, msgs: list):
        self.encoders.refresh()
        super().handle_many(msgs)


def start_proxy_visual_process(args_dict: dict, pipe_writer=None):
    import pickle as _p

    from ...models.base import embed_row_width, load_config
    from ..embed_cache.manager import EmbedCacheClient
    from ..router.manager import zmq_addr

    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::visual_proxy_server")
    start_parent_check_thread()
    try:
        assert args.config_server_host and args.config_server_port, \
            "--visual_use_proxy_mode needs --config_server_host / --config_server_port (where the encoders register)"
        cfg = getattr(args, "_config_override", None) or load_config(args.model_dir)
        ctx = zmq.Context(2)
        pull = ctx.socket(zmq.PULL)
        pull.bind(zmq_addr(args, args.visual_port))
        push = ctx.socket(zmq.PUSH)
        nxt = args.audio_port if getattr(args, "enable_multimodal_audio", False) else args.router_port
        push.connect(zmq_addr(args, nxt))
        cache = EmbedCacheClient(args, hidden=embed_row_width(cfg), open_arena=True)

        def try_recv():
            try:
                return pull.recv_pyobj(zmq.NOBLOCK)
            except zmq.ZMQError:
                return None

        mgr = ProxyVisualManager(args, cache, lambda m: push.send_pyobj(m, protocol=_p.HIGHEST_PROTOCOL),
                                 pull.recv_pyobj, infer_batch_size=args.visual_infer_batch_size or 8,
                                 try_recv=try_recv, send_batch_size=getattr(args, "visual_send_batch_size", 1) or 1)
        mgr.shm_req_manager = open_req_table(args)
    except Exception:
        if pipe_writer is not None:
            pipe_writer.send(("init failed", traceback.format_exc()))
        raise
    if pipe_writer is not None:
        pipe_writer.send("init ok")
    mgr.loop()
