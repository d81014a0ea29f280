"""Offline (in-process) engine: the public Python API for batch generation.

    llm = LLM(config=cfg_dict)                       # or LLM(model_dir="/path/to/hf/model")
    outs = llm.generate([[1, 2, 3], [4, 5]], {"max_new_tokens": 16})

It wires the same pieces the server uses, in one process per GPU: the router's Past-Future
admission queue, the per-rank `ModelBackend` (radix prefix cache, chunked prefill, decode CUDA
graphs, on-device sampling) and the model.  Under torchrun every rank constructs the same `LLM`
and calls `generate` with the same arguments; the ranks run the same schedule in lock step.
"""
from __future__ import annotations

import time
from types import SimpleNamespace
from typing import Dict, List, Optional, Union

import numpy as np
import torch

from ..models.base import load_config
from ..models.registry import get_model
from ..parallel import dist as pdist
from ..server.core.objs.req import Req
from ..server.router.req_queue import Batch, ChunkedPrefillQueue, RouterStatics
from .backend import BackendArgs, ModelBackend


class LLM:
    def __init__(self, model_dir: Optional[str] = None, config: Optional[dict] = None,
                 max_total_token_num: Optional[int] = None, running_max_req_size: int = 256,
                 batch_max_tokens: int = 16384, chunked_prefill_size: Optional[int] = None,
                 max_req_total_len: int = 8192, router_token_ratio: float = 0.85, eos_ids=(),
                 disable_dynamic_prompt_cache: bool = False, disable_cudagraph: bool = False,
                 graph_max_batch_size: Optional[int] = None, mem_fraction: float = 0.9, data_type: Optional[str] = None,
                 pstate=None, **model_kw):
        self.ps = pstate or pdist.state()
        if config is None:
            config = load_config(model_dir)
        self.config = config
        if not eos_ids:
            e = config.get("eos_token_id")
            eos_ids = tuple(e) if isinstance(e, (list, tuple)) else ((e,) if e is not None else ())
        cache_kw = dict(cpu_cache_bytes=int(model_kw.pop("cpu_cache_bytes", 0)),
                        cpu_cache_page_tokens=int(model_kw.pop("cpu_cache_page_tokens", 256)),
                        disk_cache_dir=model_kw.pop("disk_cache_dir", None),
                        disk_cache_bytes=int(model_kw.pop("disk_cache_bytes", 0)),
                        linear_att_hash_page_size=int(model_kw.pop("linear_att_hash_page_size", 512)),
                        state_host_cache_bytes=int(model_kw.pop("state_host_cache_bytes", 0)))
        tp_fused = model_kw.pop("tp_fused", None)
        no_pipeline = bool(model_kw.pop("disable_prefill_pipeline", False))
        if tp_fused is None and self.ps.tp_size > 1 and self.ps.device.type == "cuda" \
                and not model_kw.pop("disable_fused_tp", False):
            from ..parallel.fused import FusedTP

            hidden = config.get("hidden_size") or config.get("text_config", {}).get("hidden_size")
            tp_fused = FusedTP(self.ps, max_tokens=batch_max_tokens, hidden=hidden)
        self.model = get_model(config, model_dir=model_dir, pstate=self.ps, data_type=data_type, tp_fused=tp_fused,
                               max_total_token_num=max_total_token_num, mem_fraction=mem_fraction,
                               max_req_num=running_max_req_size, max_seq_length=max_req_total_len + 8,
                               batch_max_tokens=batch_max_tokens, disable_cudagraph=disable_cudagraph,
                               graph_max_batch_size=graph_max_batch_size or running_max_req_size,
                               graph_max_len_in_batch=max_req_total_len + 8, **model_kw)
        if tp_fused is not None and not no_pipeline:
            from ..parallel import ce as _ce

            _ce.attach(self.model, self.ps, batch_max_tokens, log=None)
        self.args = BackendArgs(batch_max_tokens=batch_max_tokens,
                                chunked_prefill_size=chunked_prefill_size or max(batch_max_tokens // 2, 1),
                                eos_ids=tuple(eos_ids), max_req_total_len=max_req_total_len,
                                disable_dynamic_prompt_cache=disable_dynamic_prompt_cache,
                                **cache_kw)
        if self.ps.dp_size > 1:
            from .dp_backend import DPBackend

            self.backend = DPBackend(self.model, self.args, is_master_in_dp=self.ps.tp_rank == 0)
        else:
            self.backend = ModelBackend(self.model, self.args, is_master_in_dp=True)
        self.statics = RouterStatics()
        self.queue = ChunkedPrefillQueue(max_total_tokens=self.model.max_total_token_num,
                                         batch_max_tokens=batch_max_tokens, running_max_req_size=running_max_req_size,
                                         router_token_ratio=router_token_ratio, statics=self.statics)
        self.running_max_req_size = running_max_req_size
        self._next_id = 0

    def _new_req(self, ids: List[int], params: dict) -> Req:
        r = Req()
        r.index_in_shm_mem = -1
        rid = self._next_id
        self._next_id += 8
        r.init(rid, ids, params, None, chunked_prefill_size=self.args.chunked_prefill_size,
               router_max_wait_tokens=self.args.router_max_wait_tokens, max_total_len=self.args.max_req_total_len)
        rc = getattr(self.model, "route_capture", None)
        if rc is not None:
            r.create_routed_shm_array(rc.num_layers, rc.top_k, rc.np_dtype)
        return r

    def warmup(self, batch_sizes: Optional[List[int]] = None):
        from ..utils import autotuner

        if autotuner.autotune_level() > 0 and self.model.device.type == "cuda" and self.config.get("intermediate_size"):
            # tune the GEMM variants of this model's shapes before the decode graphs capture their choices
            sizes = sorted(set(batch_sizes or self.model.graph_batch_sizes()))
            pick = sorted({sizes[0], sizes[-1], *sizes[:: max(1, len(sizes) // 6)]})
            autotuner.tune_model(self.config, self.ps.tp_size, Ms=pick, group=self.ps.cpu_group,
                                 force=autotuner.autotune_level() >= 2, log=None)
        self.model.warmup_graphs(batch_sizes)

    def close(self):
        """Release captured graphs (they hold the process group's collectives) and the peer-mapped buffers; call
        before tearing the process group down."""
        if self.model.device.type == "cuda":
            torch.cuda.synchronize(self.model.device)
        self.model.flush_graphs()
        fused = getattr(self.model.tp, "fused", None)
        ce = getattr(self.model.tp, "ce", None)
        if ce is not None:
            self.model.tp.ce = None
            ce.close()
        if fused is not None:
            fused.check()
            self.model.tp.fused = None
            fused.close()

    def _arrived(self, arrival_times, t_start: float, n_in: int) -> int:
        """How many requests have arrived by now.  With several ranks the first rank's clock decides and the
        others are told (one small host broadcast per scheduling round), so that all ranks admit the same
        requests on the same step."""
        n = n_in
        if self.ps.global_rank == 0 or self.ps.world_size == 1:
            now = time.time() - t_start
            while n < len(arrival_times) and arrival_times[n] <= now:
                n += 1
        if self.ps.world_size > 1 and self.ps.cpu_group is not None:
            import torch.distributed as dist

            t = torch.tensor([n], dtype=torch.int64)
            dist.broadcast(t, src=0, group=self.ps.cpu_group)
            n = int(t.item())
        return n

    @torch.no_grad()
    def generate(self, prompt_token_ids: List[List[int]], sampling_params: Union[dict, List[dict], None] = None,
                 return_stats: bool = False, arrival_times: Optional[List[float]] = None):
        """Runs every prompt to completion with continuous batching; returns one dict per prompt:
        {"token_ids", "logprobs", "finish_reason", "prompt_tokens", "ttft_s", "latency_s"}.
        `arrival_times` (seconds from the call, non-decreasing): request i only enters the admission queue once its
        time has come (an open-loop load, e.g. Poisson arrivals); "ttft_s" and "latency_s" then count from the
        request's own arrival."""
        n = len(prompt_token_ids)
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params or {}] * n
        reqs = []
        limit = self.args.max_req_total_len
        for ids, sp in zip(prompt_token_ids, sampling_params):
            sp = dict(sp)
            if len(ids) + 1 > limit:
                raise ValueError(f"prompt of {len(ids)} tokens exceeds max_req_total_len {limit}")
            sp["max_new_tokens"] = min(sp.get("max_new_tokens", 16), limit - len(ids))
            reqs.append(self._new_req(list(ids), sp))
        t_submit = time.time()
        timed = arrival_times is not None
        if timed:
            assert len(arrival_times) == n and self.ps.dp_size == 1, "timed arrivals: one time per prompt, no --dp"
            n_in = 0
        else:
            self.queue.extend(reqs)
        running = Batch(0, [])
        done = 0
        finish_time: Dict[int, float] = {}
        token_times: Dict[int, list] = {r.request_id: [] for r in reqs} if return_stats else None
        if return_stats:
            self.backend.on_token = lambda ir, tok, lp: token_times[ir.req_id].append(time.time())
        step_log = []
        while done < n:
            if timed and n_in < n:
                upto = self._arrived(arrival_times, t_submit, n_in)
                if upto > n_in:
                    self.queue.extend(reqs[n_in:upto])
                    n_in = upto
                if not self.backend.has_work() and self.queue.get_wait_req_num() == 0:
                    time.sleep(0.0005)   # nothing running, nothing waiting: the next request has not arrived yet
                    continue
            used = 1.0 - self.backend.ctx.get_can_alloc_token_num() / max(self.model.max_total_token_num, 1)
            self.queue.cur_token_usage_ratio = used
            new_batch = self.queue.generate_new_batch(running)
            if new_batch is not None:
                self.backend.add_reqs(new_batch.reqs)
                running.merge(new_batch)
            if not self.backend.has_work():
                if self.queue.get_wait_req_num() == 0:
                    break
                raise RuntimeError("scheduler stalled: waiting requests do not fit the KV pool")
            res = self.backend.step()
            if return_stats:
                step_log.append((res["kind"], res["tokens"]))
            for ir in res["finished"]:
                done += 1
                finish_time[ir.req_id] = time.time()
                self.statics.update(ir.cur_output_len)
            running.filter_out_finished_req()
        self.backend.on_token = None
        outs = []
        for i, r in enumerate(reqs):
            out_ids = r.get_output_ids()
            lps = r.shm_logprobs.arr[r.input_len: r.input_len + r.shm_cur_output_len].tolist()
            t_arrive = t_submit + (arrival_times[i] if timed else 0.0)
            o = {"token_ids": out_ids, "logprobs": lps, "finish_reason": r.finish_status.get_finish_reason(),
                 "prompt_tokens": r.input_len, "prompt_cache_len": r.prompt_cache_len,
                 "ttft_s": (r.first_token_time - t_arrive) if r.first_token_time > 0 else None,
                 "latency_s": finish_time.get(r.request_id, time.time()) - t_arrive}
            if return_stats:
                o["token_times"] = token_times[r.request_id]
            if getattr(r, "shm_routed", None) is not None:
                o["routed_experts"] = r.shm_routed.arr[:r.routed_len].copy()
            outs.append(o)
            r.release_shm_arrays()
        if hasattr(self.backend, "drain"):
            self.backend.drain()
        if return_stats:
            return outs, {"steps": step_log, "backend": dict(self.backend.stats)}
        return outs
