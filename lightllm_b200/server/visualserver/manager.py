"""visual server process: sits between the HTTP workers and the router for multimodal deployments.  It pulls
`GroupReqIndexes` from the HTTP workers, embeds the images that the embed cache does not hold yet (batched
through the model's vision tower, on its own GPU stream / device), writes the embeddings into the shared arena,
marks them ready and forwards the request to the next stage (audio server or router).  Requests without
images pass straight through.  `--visual_dp` towers work on disjoint image subsets in parallel threads.
Reference: lightllm/server/visualserver/manager.py, model_infer/model_rpc.py.
"""
from __future__ import annotations

import pickle
import time
import traceback
from typing import List

import torch
import zmq

from ...utils.process_utils import set_proc_title, start_parent_check_thread
from ..core.objs.io_objs import GroupReqIndexes
from ..core.objs.start_args import StartArgs
from ..embed_cache.manager import EmbedCacheClient


def build_vision_tower(args, device, dtype=torch.bfloat16):
    """The vision tower of the served model (by `model_type`)."""
    from ...models.base import load_config
    from ...models.weights import RandomSource, SafetensorsSource

    cfg = getattr(args, "_config_override", None) or load_config(args.model_dir)
    mt = cfg.get("model_type")
    from ...models.qwen2_vl import is_tarsier2

    tarsier2 = is_tarsier2(cfg)
    if mt in ("qwen2_vl", "qwen2_5_vl") or tarsier2:
        from ...models.base import TransformerLM
        from ...models.vit.qwen2_vl_visual import Qwen2VLVisionTower

        vcfg = dict(cfg["vision_config"])
        vcfg.setdefault("hidden_size", cfg["hidden_size"])
        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(Qwen2VLVisionTower.weight_shapes(vcfg), dtype=dtype)
        # Tarsier2 keeps the same tower under `vision_tower.`
        prefix = "vision_tower." if tarsier2 and src.has("vision_tower.patch_embed.proj.weight") else None
        return Qwen2VLVisionTower(vcfg, src, device, dtype, prefix=prefix)
    if mt in ("qwen3_vl", "qwen3_vl_moe", "qwen3_5", "qwen3_5_moe"):
        from ...models.base import TransformerLM
        from ...models.vit.qwen3_vl_visual import Qwen3VLVisionTower

        vcfg = dict(cfg["vision_config"])
        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(Qwen3VLVisionTower.weight_shapes(vcfg), dtype=dtype)
        return Qwen3VLVisionTower(vcfg, src, device, dtype)
    if mt == "qwen" and "visual" in cfg:
        from ...models.base import TransformerLM
        from ...models.vit.qwen_vl_visual import QwenVLVisionTower

        vcfg = dict(cfg["visual"])
        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(QwenVLVisionTower.weight_shapes(vcfg), dtype=dtype)
        return QwenVLVisionTower(vcfg, src, device, dtype)
    if mt == "qwen3_omni_moe":
        from ...models.base import TransformerLM
        from ...models.qwen3_omni import Qwen3OmniVisionTower

        vcfg = dict(cfg["vision_config"])
        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(Qwen3OmniVisionTower.weight_shapes(vcfg), dtype=dtype)
        return Qwen3OmniVisionTower(vcfg, src, device, dtype)
    if mt == "llava":
        from ...models.vit.clip_visual import ClipLlavaTower

        return ClipLlavaTower(cfg, SafetensorsSource(args.model_dir), device, dtype)
    if mt == "gemma4":
        from ...models.vit.gemma4_visual import Gemma4VisionTower

        return Gemma4VisionTower(cfg, SafetensorsSource(args.model_dir), device, dtype)
    if mt == "gemma3":
        from ...models.vit.siglip_visual import SiglipGemma3Tower

        return SiglipGemma3Tower(cfg, SafetensorsSource(args.model_dir), device, dtype)
    if mt == "internvl_chat":
        from ...models.base import TransformerLM
        from ...models.vit.internvl_visual import InternVLVisionTower

        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(InternVLVisionTower.weight_shapes(cfg), dtype=dtype)
        return InternVLVisionTower(cfg, src, device, dtype)
    raise ValueError(f"no vision tower for model_type {mt!r}")


def encode_on_replicas(towers, n_items: int, batch_size: int, encode):
    """Data-parallel encoder pass: the item indices 0..n_items-1 are dealt round-robin to the towers, every tower
    works through its share in batches of `batch_size` on a thread of its own (bound to the tower's GPU), and
    `encode(tower, indices) -> list of tensors` does one batch.  Returns the results by item index."""
    from concurrent.futures import ThreadPoolExecutor

    out = [None] * n_items

    def work(r):
        tower = towers[r]
        dev = getattr(tower, "device", None)
        if dev is not None and getattr(dev, "type", "cpu") == "cuda":
            torch.cuda.set_device(dev)
        mine = list(range(r, n_items, len(towers)))
        for s in range(0, len(mine), batch_size):
            idx = mine[s:s + batch_size]
            for i, e in zip(idx, encode(tower, idx)):
                out[i] = e

    with ThreadPoolExecutor(max_workers=len(towers)) as ex:
        list(ex.map(work, range(len(towers))))
    return out


def replica_devices(gpu_ids, dp: int):
    """One device per encoder replica: `gpu_ids[r]` (cycled when fewer are given), the CPU without CUDA."""
    dp = max(1, int(dp or 1))
    if not torch.cuda.is_available():
        return [torch.device("cpu")] * dp
    ids = list(gpu_ids or range(dp))
    return [torch.device("cuda", ids[r % len(ids)]) for r in range(dp)]


class VisualManager:
    def __init__(self, args: StartArgs, tower=None, cache=None, send_next=None, recv=None, infer_batch_size: int = 8,
                 try_recv=None, send_batch_size: int = 1, towers=None):
        self.args = args
        self.towers = list(towers) if towers else ([tower] if tower is not None else [])   # `--visual_dp` replicas
        tower = self.towers[0] if self.towers else None
        self.tower = tower
        self.cache = cache
        self.send_next = send_next
        self.recv = recv
        self.try_recv = try_recv                  # non-blocking receive (None when nothing waits)
        self.send_batch_size = max(1, int(send_batch_size or 1))   # `--visual_send_batch_size`
        self.infer_batch_size = infer_batch_size
        self.waiting: List[GroupReqIndexes] = []

    def _pending_images(self, group: GroupReqIndexes):
        mm = group.multimodal_params or {}
        imgs = mm.get("images", []) if isinstance(mm, dict) else []
        if not imgs:
            return []
        ready = self.cache.get_items_embed([i["uuid"] for i in imgs])
        return [i for i, r in zip(imgs, ready) if not r]

    def embed(self, images: List[dict]):
        """Runs the tower over `images` (deduplicated by cache record) and publishes the embeddings."""
        uniq = {i["uuid"]: i for i in images}
        items = list(uniq.values())
        if len(self.towers) > 1 and len(items) > 1:
            # the cache client is one socket: payloads are read and results written on this thread, only the
            # tower passes run side by side
            payloads = [self.cache.get_payload(i["uuid"]) for i in items]
            embs = encode_on_replicas(self.towers, len(items), self.infer_batch_size, lambda tower, idx: tower.encode_images(
                [payloads[i] for i in idx], items=[items[i] for i in idx]))
            for it, e in zip(items, embs):
                assert e.shape[0] == it["token_num"], f"image gives {e.shape[0]} tokens, the prompt reserved {it['token_num']}"
                self.cache.arena.write(it["start_index_in_embed_cache"], e)
            self.cache.set_items_embed([i["uuid"] for i in items])
            return
        for s in range(0, len(items), self.infer_batch_size):
            chunk = items[s:s + self.infer_batch_size]
            payloads = [self.cache.get_payload(i["uuid"]) for i in chunk]
            embs = self.tower.encode_images(payloads, items=chunk)
            for it, e in zip(chunk, embs):
                assert e.shape[0] == it["token_num"], f"image gives {e.shape[0]} tokens, the prompt reserved {it['token_num']}"
                self.cache.arena.write(it["start_index_in_embed_cache"], e)
            self.cache.set_items_embed([i["uuid"] for i in chunk])

    def handle(self, group: GroupReqIndexes):
        pending = self._pending_images(group)
        if pending:
            self.embed(pending)
        self.send_next(group)

    def handle_many(self, msgs: list):
        """Requests that arrived together share encoder passes: their missing pictures are embedded in batches of
        `infer_batch_size` (one record once, however many requests carry it), then everything travels on in arrival
        order (control commands keep their place).  When the pass fails, the requests whose pictures are still
        missing are marked aborted before they travel on: the router ends them instead of running them over
        unwritten arena rows."""
        failed = set()
        pending = []
        for m in msgs:
            if isinstance(m, GroupReqIndexes):
                pending += self._pending_images(m)
        if pending:
            try:
                self.embed(pending)
            except Exception:
                traceback.print_exc()
                for m in msgs:
                    try:
                        if isinstance(m, GroupReqIndexes) and self._pending_images(m):
                            failed.add(id(m))
                    except Exception:
                        failed.add(id(m))
        for m in msgs:
            if id(m) in failed:
                self._abort(m)
            self.send_next(m)

    def _abort(self, group: GroupReqIndexes):
        mgr = getattr(self, "shm_req_manager", None)
        if mgr is None:
            return
        for idx in group.shm_req_indexes:
            req = mgr.get_req_obj_by_index(idx)
            req.is_aborted = True
            mgr.put_back_req_obj(req)

    def loop(self):
        while True:
            msgs = [self.recv()]
            while self.try_recv is not None and len(msgs) < self.send_batch_size:
                m = self.try_recv()
                if m is None:
                    break
                msgs.append(m)
            self.handle_many(msgs)


def open_req_table(args):
    """The shared request table, to mark requests aborted; None where there is none (a tower used on its own)."""
    try:
        from ..core.objs.shm_req_manager import ShmReqManager
        from ..core.objs.start_args import set_env_start_args

        set_env_start_args(args)
        return ShmReqManager(args.unique_server_name, args.running_max_req_size)
    except Exception:
        traceback.print_exc()
        return None


def start_visual_process(args_dict: dict, pipe_writer=None):
    from ..router.manager import zmq_addr

    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::visual_server")
    start_parent_check_thread()
    try:
        towers = [build_vision_tower(args, dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
                  for dev in replica_devices(args.visual_gpu_ids, getattr(args, "visual_dp", 1))]
        tower = towers[0]
        ctx = zmq.Context(2)
        pull = ctx.socket(zmq.PULL)
        pull.bind(zmq_addr(args, args.visual_port))
        push = ctx.socket(zmq.PUSH)
        nxt = args.audio_port if getattr(args, "enable_multimodal_audio", False) else args.router_port
        push.connect(zmq_addr(args, nxt))
        cache = EmbedCacheClient(args, hidden=tower.out_hidden, open_arena=True)
        def try_recv():
            try:
                return pull.recv_pyobj(zmq.NOBLOCK)
            except zmq.ZMQError:
                return None

        mgr = VisualManager(args, tower, cache, lambda m: push.send_pyobj(m, protocol=pickle.HIGHEST_PROTOCOL),
                            pull.recv_pyobj, infer_batch_size=args.visual_infer_batch_size or 8, try_recv=try_recv,
                            send_batch_size=getattr(args, "visual_send_batch_size", 1) or 1, towers=towers)
        mgr.shm_req_manager = open_req_table(args)
    except Exception:
        if pipe_writer is not None:
            pipe_writer.send(("init failed", traceback.format_exc()))
        raise
    if pipe_writer is not None:
        pipe_writer.send("init ok")
    mgr.loop()
