"""Audio server process: sits between the visual server (or the HTTP workers) and the router.  For every request
group with audio clips whose embeddings are not in the embed cache yet it reads the decoded PCM payload from the
cache, runs the Whisper tower + projector, writes the embeddings into the shared arena and marks the records
ready; then the group travels on to the router.  Reference: lightllm/server/audioserver/manager.py.
"""
from __future__ import annotations

import pickle
import traceback
from typing import List

import numpy as np
import torch
import zmq

from ...utils.process_utils import set_proc_title, start_parent_check_thread
from ..core.objs.io_objs import GroupReqIndexes
from ..core.objs.start_args import StartArgs
from ..embed_cache.manager import EmbedCacheClient


def build_audio_tower(args, device, dtype=torch.bfloat16):
    from ...models.base import TransformerLM, load_config
    from ...models.weights import RandomSource, SafetensorsSource
    from ...models.whisper_audio import WhisperAudioTower

    cfg = getattr(args, "_config_override", None) or load_config(args.model_dir)
    if "audio_config" not in cfg:
        raise ValueError(f"model_type {cfg.get('model_type')!r} has no audio tower (no audio_config)")
    if cfg.get("model_type") == "qwen3_omni_moe":
        from ...models.qwen3_omni import Qwen3OmniAudioTower

        if args.model_dir and TransformerLM._has_weights(args.model_dir):
            src = SafetensorsSource(args.model_dir)
        else:
            src = RandomSource(Qwen3OmniAudioTower.weight_shapes(cfg), dtype=dtype)
        return Qwen3OmniAudioTower(cfg, src, device, dtype)
    if args.model_dir and TransformerLM._has_weights(args.model_dir):
        src = SafetensorsSource(args.model_dir)
    else:
        src = RandomSource(WhisperAudioTower.weight_shapes(cfg), dtype=dtype)
    return WhisperAudioTower(cfg, src, device, dtype)


class AudioManager:
    def __init__(self, args: StartArgs, tower=None, cache=None, send_next=None, recv=None, infer_batch_size: int = 8,
                 towers=None):
        self.towers = list(towers) if towers else ([tower] if tower is not None else [])      # `--audio_dp` replicas
        tower = self.towers[0] if self.towers else None
        self.args, self.tower, self.cache = args, tower, cache
        self.shm_req_manager = None
        self.send_next, self.recv = send_next, recv
        self.infer_batch_size = infer_batch_size

    def _pending(self, group: GroupReqIndexes):
        mm = group.multimodal_params or {}
        auds = mm.get("audios", []) if isinstance(mm, dict) else []
        if not auds:
            return []
        ready = self.cache.get_items_embed([a["uuid"] for a in auds])
        return [a for a, r in zip(auds, ready) if not r]

    def embed(self, audios: List[dict]):
        items = list({a["uuid"]: a for a in audios}.values())
        for s in range(0, len(items), self.infer_batch_size * max(1, len(self.towers))):
            chunk = items[s:s + self.infer_batch_size * max(1, len(self.towers))]
            clips = [np.frombuffer(self.cache.get_payload(a["uuid"]), dtype=np.float32) for a in chunk]
            if len(self.towers) > 1 and len(chunk) > 1:
                from ..visualserver.manager import encode_on_replicas

                embs = encode_on_replicas(self.towers, len(chunk), self.infer_batch_size, lambda tower, idx: tower.encode_audios(
                    [clips[i] for i in idx], items=[chunk[i] for i in idx]))
            else:
                embs = self.tower.encode_audios(clips, items=chunk)
            for it, e in zip(chunk, embs):
                assert e.shape[0] == it["token_num"], f"clip gives {e.shape[0]} tokens, the prompt reserved {it['token_num']}"
                arr = getattr(self.cache.arena, "arr", None)
                width = arr.shape[1] if arr is not None else e.shape[1]
                if e.shape[1] < width:  # arena rows also hold deep-stack image features: zeros for audio
                    e = torch.nn.functional.pad(e, (0, width - e.shape[1]))
                self.cache.arena.write(it["start_index_in_embed_cache"], e)
            self.cache.set_items_embed([a["uuid"] for a in chunk])

    def handle(self, group: GroupReqIndexes):
        pending = self._pending(group)
        if pending:
            self.embed(pending)
        self.send_next(group)

    def loop(self):
        while True:
            msg = self.recv()
            try:
                if isinstance(msg, GroupReqIndexes):
                    self.handle(msg)
                else:
                    self.send_next(msg)
            except Exception:
                traceback.print_exc()
                # clips that could not be embedded: their requests end as aborted instead of running over
                # unwritten arena rows
                if isinstance(msg, GroupReqIndexes) and self.shm_req_manager is not None:
                    for idx in msg.shm_req_indexes:
                        req = self.shm_req_manager.get_req_obj_by_index(idx)
                        req.is_aborted = True
                        self.shm_req_manager.put_back_req_obj(req)
                self.send_next(msg)


def start_audio_process(args_dict: dict, pipe_writer=None):
    from ..router.manager import zmq_addr

    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::audio_server")
    start_parent_check_thread()
    try:
        from ..visualserver.manager import open_req_table, replica_devices

        gpu_ids = getattr(args, "audio_gpu_ids", None) or args.visual_gpu_ids
        towers = [build_audio_tower(args, dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
                  for dev in replica_devices(gpu_ids, getattr(args, "audio_dp", 1))]
        tower = towers[0]
        ctx = zmq.Context(2)
        pull = ctx.socket(zmq.PULL)
        pull.bind(zmq_addr(args, args.audio_port))
        push = ctx.socket(zmq.PUSH)
        push.connect(zmq_addr(args, args.router_port))
        cache = EmbedCacheClient(args, hidden=tower.out_hidden, open_arena=True)
        mgr = AudioManager(args, tower, cache, lambda m: push.send_pyobj(m, protocol=pickle.HIGHEST_PROTOCOL),
                           pull.recv_pyobj, infer_batch_size=int(getattr(args, "audio_infer_batch_size", 0) or 8),
                           towers=towers)
        mgr.shm_req_manager = open_req_table(args)
    except Exception:
        if pipe_writer is not None:
            pipe_writer.send(("init failed", traceback.format_exc()))
        raise
    if pipe_writer is not None:
        pipe_writer.send("init ok")
    mgr.loop()
