"""Request front-end inside each HTTP worker process.

`generate()` is the async generator every API route consumes: it tokenises, validates and
repairs lengths, allocates shm request slots, writes the request, pushes the slot indices to the
router, then yields `(sub_req_id, text, metadata, FinishStatus)` as the detokenizer fills the
request's output ring.  `handle_loop()` wakes on the detokenizer's zmq PUB tick (or every 50 ms)
and drains the rings of all live requests; `recycle_resource_loop()` returns finished slots.

Reference: lightllm/server/httpserver/manager.py:47-986.
"""
from __future__ import annotations

import asyncio
import pickle
import time
from typing import Dict, List, Optional, Union

import zmq
import zmq.asyncio

from ...utils.errors import ServerBusyError
from ..core.objs.atomic_lock import SharedInt
from ..core.objs.io_objs import FlushCacheCmd, GroupReqIndexes, ProfilerCmd, RLCmd
from ..core.objs.req import FinishStatus, Req
from ..core.objs.sampling_params import SamplingParams
from ..core.objs.shm_req_manager import ShmReqManager
from ..core.objs.start_args import StartArgs
from ..req_id_generator import ReqIDGenerator, convert_sub_id_to_group_id
from ..tokenizer import get_tokenizer


class ReqStatus:
    def __init__(self, group_req_id: int, multimodal_params, req_objs: List[Req], start_time: float):
        self.lock = asyncio.Lock()
        self.event = asyncio.Event()
        self.group_req_id = group_req_id
        self.multimodal_params = multimodal_params
        self.req_objs = req_objs
        self.start_time = start_time
        self.out_token_info_list: List[tuple] = []
        self.finished = set()

    def can_release(self) -> bool:
        return all(r.can_release() for r in self.req_objs)


class HttpServerManager:
    def __init__(self, args: StartArgs, metric_client=None):
        from ..router.manager import zmq_addr

        self.args = args
        self.name = args.unique_server_name
        ctx = zmq.asyncio.Context(2)
        self.send_to_router = ctx.socket(zmq.PUSH)
        self.send_to_router.connect(zmq_addr(args, args.router_port))
        self.recv_from_detok = ctx.socket(zmq.SUB)
        self.recv_from_detok.connect(zmq_addr(args, args.http_server_port))
        self.recv_from_detok.setsockopt(zmq.SUBSCRIBE, b"")
        self.shm_req_manager = ShmReqManager(self.name, args.running_max_req_size)
        self.tokenizer = get_tokenizer(args.model_dir, args.tokenizer_mode, args.trust_remote_code, args.vocab_size,
                                       multimodal=bool(getattr(args, "enable_multimodal", False)),
                                       config_override=getattr(args, "_config_override", None))
        self.enable_multimodal = bool(getattr(args, "enable_multimodal", False))
        self.embed_cache = None
        if self.enable_multimodal:
            from ..embed_cache.manager import EmbedCacheClient

            self.embed_cache = EmbedCacheClient(args)
            self.send_to_visual = ctx.socket(zmq.PUSH)
            self.send_to_visual.connect(zmq_addr(args, args.visual_port))
        self.vocab_size = args.vocab_size
        self.id_gen = ReqIDGenerator(self.name)
        self.req_id_to_out_inf: Dict[int, ReqStatus] = {}
        self.max_req_total_len = args.max_req_total_len
        self.shm_max_total_token_num = SharedInt(f"{self.name}_max_total_token_num")
        self.latest_success_infer_time_mark = SharedInt(f"{self.name}_latest_success_infer_time_mark")
        self.latest_success_infer_time_mark.set_value(int(time.time()))
        self.run_reqs_count_mark = SharedInt(f"{self.name}_run_reqs_count_mark")
        self.metric_client = metric_client
        self.paused = False  # RL: admission gate
        self.routed_shape = None  # (MoE layers, top_k, dtype) with --enable_return_routed_experts
        if getattr(args, "enable_return_routed_experts", False):
            from ...common import route_capture as rc
            from ...models.base import load_config

            cfg = getattr(args, "_config_override", None) or load_config(args.model_dir)
            if not rc.moe_layer_map(cfg):
                raise ValueError("--enable_return_routed_experts needs a mixture-of-experts model")
            self.routed_shape = (len(rc.moe_layer_map(cfg)), rc.top_k_of(cfg), rc.np_dtype_of(cfg))
        self.relay_master = None  # httpserver/multinode_relay.py on node 0 of a multi-node tensor-parallel deployment
        self.master_id_to_local: Dict[int, int] = {}  # PD nodes: pd_master request id -> local group id
        self.eos_ids = set(args.eos_ids or [])
        self.all_special_ids = set(getattr(self.tokenizer, "all_special_ids", []) or [])
        self._recycle_event = asyncio.Event()

    # ------------------------------------------------------------------ helpers
    def tokens(self, prompt: str, multimodal_params=None, samping_params=None, kwargs=None) -> int:
        return len(self.tokenizer.encode(prompt, **(kwargs or {})))

    async def _alloc_multimodal(self, mm, sampling_params):
        """Cache records for every image / audio clip: token-id ranges and arena rows; new payloads are uploaded
        for the visual / audio server.  Retries while the cache is full of referenced records."""
        items = mm.items()
        md5s, nums = [], []
        for it in items:
            init = getattr(self.tokenizer, "init_imageitem_extral_params" if it.kind == "image"
                           else "init_audioitem_extral_params", None)
            if init is not None:  # per-item settings that change the token count (e.g. the tile budget of an image)
                init(it, mm, sampling_params)
            n = self.tokenizer.get_image_token_length(it) if it.kind == "image" else \
                self.tokenizer.get_audio_token_length(it)
            cap = int(getattr(self.args, "max_image_token_count", 0) or 0)
            if it.kind == "image" and cap > 0 and n > cap:
                raise ValueError(f"an image needs {n} tokens, --max_image_token_count allows {cap}")
            it.token_num = n
            it.md5 = it.content_md5(salt=str(getattr(it, "grid_thwd", "")) + str(sorted(it.extra_params.items())))
            md5s.append(it.md5)
            nums.append(n)
        t0 = time.time()
        while True:
            recs = self.embed_cache.alloc(md5s, nums)
            if recs is not None:
                break
            if time.time() - t0 > 30:
                raise ServerBusyError("the multimodal embedding cache is full")
            await asyncio.sleep(0.05)
        have = self.embed_cache.get_items_data([r["id"] for r in recs])
        new_ids, payloads = [], []
        for it, r, h in zip(items, recs, have):
            it.uuid, it.token_id, it.start_index_in_embed_cache = r["id"], r["token_id"], r["start_index_in_embed_cache"]
            data = it.read()
            if not h and r["id"] not in new_ids:
                new_ids.append(r["id"])
                payloads.append(data)
        if new_ids:
            self.embed_cache.set_items_data(new_ids, payloads)
        return [r["id"] for r in recs]

    async def _encode(self, prompt: Union[str, List[int]], sampling_params: SamplingParams, mm=None):
        if mm is not None:  # text or token ids with image placeholders: the wrapper expands the placeholders
            loop = asyncio.get_running_loop()
            return list(await loop.run_in_executor(None, lambda: self.tokenizer.encode(
                prompt, mm, add_special_tokens=sampling_params.add_special_tokens)))
        if isinstance(prompt, str):
            loop = asyncio.get_running_loop()
            ids = await loop.run_in_executor(None, lambda: self.tokenizer.encode(
                prompt, add_special_tokens=sampling_params.add_special_tokens))
            return list(ids)
        ids = list(prompt)
        if self.vocab_size is not None and any((not isinstance(t, int)) or t < 0 or t >= self.vocab_size for t in ids):
            raise ValueError("prompt token ids must be integers inside the vocabulary")
        return ids

    def _check_and_repair_length(self, prompt_ids: List[int], sp: SamplingParams, multimodal: bool = False):
        """max_new_tokens is clamped so that prompt + output fits the pool and the per-request limit."""
        if not prompt_ids:
            raise ValueError("prompt must not be empty")
        pool = self.shm_max_total_token_num.get_value()
        limit = self.max_req_total_len if pool <= 0 else min(pool - 36, self.max_req_total_len)
        n = len(prompt_ids)
        if n + 1 > limit:
            raise ValueError(f"the prompt has {n} tokens, the limit for prompt + output is {limit}")
        if n + sp.max_new_tokens > limit:
            sp.max_new_tokens = limit - n
            sp.min_new_tokens = min(sp.min_new_tokens, sp.max_new_tokens)
        return prompt_ids

    # ------------------------------------------------------------------ generate
    async def generate(self, prompt: Union[str, List[int]], sampling_params: SamplingParams, multimodal_params=None,
                       request=None, is_health_req: bool = False, pd_info: Optional[dict] = None,
                       group_req_id: Optional[int] = None):
        """`pd_info` (P/D nodes only) = {"group_req_id": the pd_master's id, "peer": the paired node}.
        `group_req_id`: set on the follower nodes of a multi-node tensor-parallel deployment, where node 0 chose it."""
        if self.paused and not is_health_req:
            raise ServerBusyError("generation is paused")
        start_time = time.time()
        if group_req_id is None:
            group_req_id = self.id_gen.generate_id()
        sampling_params.group_request_id = group_req_id
        mm, mm_record_ids = None, []
        if multimodal_params and self.enable_multimodal and \
                (multimodal_params.get("images") or multimodal_params.get("audios")):
            from ..multimodal_params import MultimodalParams

            mm = MultimodalParams(**multimodal_params)
            await mm.verify_and_preload(request)
            mm_record_ids = await self._alloc_multimodal(mm, sampling_params)
            multimodal_params = mm.to_dict()
        try:
            prompt_ids = await self._encode(prompt, sampling_params, mm)
            prompt_ids = self._check_and_repair_length(prompt_ids, sampling_params, multimodal=mm is not None)
        except Exception:
            if mm_record_ids:
                self.embed_cache.release(mm_record_ids)
            raise
        if pd_info is not None:
            self.master_id_to_local[pd_info["group_req_id"]] = group_req_id
            if self.args.run_mode == "prefill" and pd_info.get("peer"):
                ip, port = pd_info["peer"]["kv_endpoint"]
                sampling_params.pd_kv_trans_params.set({"peer_ip": ip, "peer_port": port,
                                                        "master_req_id": pd_info["group_req_id"],
                                                        "decode_node_id": pd_info["peer"]["node_id"],
                                                        "decode_dp": pd_info["peer"].get("dp", 1),
                                                        "decode_tp": pd_info["peer"].get("tp", 1)})
        if request is not None and not is_health_req:   # correlate with the caller's own ids in the log
            hdr = getattr(request, "headers", None) or {}
            xid, sid = hdr.get("X-Request-Id", ""), hdr.get("X-Session-Id", "")
            if xid or sid:
                print(f"[http] received req X-Request-Id:{xid} X-Session-Id:{sid} lightllm_req_id:{group_req_id}",
                      flush=True)
        if self.metric_client is not None:
            # tokenisation, multimodal preload and length checks: everything before the request can be queued
            self.metric_client.histogram_observe("lightllm_request_validation_duration", time.time() - start_time)
            self.metric_client.counter_inc("lightllm_request_count")
            self.metric_client.histogram_observe("lightllm_request_input_length", len(prompt_ids))
            self.metric_client.histogram_observe("lightllm_request_max_new_tokens", sampling_params.max_new_tokens)
        req_objs: List[Req] = []
        indexes = []
        try:
            for i in range(sampling_params.n):
                idx = await self.shm_req_manager.async_alloc_req_index()
                t0 = time.time()
                while idx is None:
                    if time.time() - t0 > 2.0:
                        raise ServerBusyError("no free request slot (running_max_req_size reached)")
                    await asyncio.sleep(0.005)
                    idx = await self.shm_req_manager.async_alloc_req_index()
                indexes.append(idx)
            for i, idx in enumerate(indexes):
                r = await self.shm_req_manager.async_get_req_obj_by_index(idx)
                r.init(group_req_id + i, prompt_ids, sampling_params, self.tokenizer,
                       chunked_prefill_size=self.args.chunked_prefill_size or 0,
                       router_max_wait_tokens=self.args.router_max_wait_tokens, mtp_step=self.args.mtp_step,
                       shm_prefix=self.name, max_total_len=self.max_req_total_len)
                r.group_req_id = group_req_id
                if self.routed_shape is not None:
                    r.create_routed_shm_array(*self.routed_shape)
                if self.args.enable_prompt_logprobs is False:
                    r.sample_params.prompt_logprobs = -1
                elif r.sample_params.prompt_logprobs >= 0:
                    r.create_prompt_meta_shm_array()
                req_objs.append(r)
        except Exception:
            for r in req_objs:
                r.release_shm_arrays(unlink=True)
                await self.shm_req_manager.async_put_back_req_obj(r)
            for idx in indexes:
                await self.shm_req_manager.async_release_req_index(idx)
            raise
        status = ReqStatus(group_req_id, multimodal_params, req_objs, start_time)
        self.req_id_to_out_inf[group_req_id] = status
        self.run_reqs_count_mark.add(1)
        first_stage = self.send_to_visual if mm is not None else self.send_to_router
        if self.relay_master is not None:     # multi-node tensor parallelism: the other nodes queue the same request
            await self.relay_master.relay(group_req_id, prompt_ids, sampling_params, multimodal_params)
        await first_stage.send_pyobj(GroupReqIndexes(group_req_id, multimodal_params, indexes, start_time),
                                     protocol=pickle.HIGHEST_PROTOCOL)
        try:
            first = True
            async for item in self._wait_to_token_package(start_time, len(prompt_ids), group_req_id, sampling_params,
                                                          status, request):
                if first and pd_info is not None and self.args.run_mode == "prefill":
                    item[2]["prompt_ids"] = prompt_ids  # the pd_master hands them to the decode node
                if first:     # only the first token's record says what the prompt was made of
                    img = sum(int(i.token_num or 0) for i in mm.images) if mm is not None else 0
                    aud = sum(int(a.token_num or 0) for a in mm.audios) if mm is not None else 0
                    item[2]["input_usage"] = {"input_text_tokens": len(prompt_ids) - img - aud,
                                              "input_audio_tokens": aud, "input_image_tokens": img}
                first = False
                yield item
        finally:
            self.run_reqs_count_mark.add(-1)
            if mm_record_ids:
                self.embed_cache.release(mm_record_ids)
            if pd_info is not None:
                self.master_id_to_local.pop(pd_info["group_req_id"], None)

    async def _wait_to_token_package(self, start_time, prompt_tokens, group_req_id, sampling_params, status: ReqStatus,
                                     request):
        unfinished = sampling_params.n
        first_token_cost = None
        out_count = 0
        is_first = True
        while True:
            try:
                await asyncio.wait_for(status.event.wait(), timeout=5)
            except asyncio.TimeoutError:
                pass
            if request is not None and await request.is_disconnected():
                await self.abort(group_req_id)
                raise asyncio.CancelledError(f"client disconnected, req {group_req_id} aborted")
            async with status.lock:
                status.event.clear()
                items, status.out_token_info_list = status.out_token_info_list, []
            for sub_req_id, text, metadata, finish_status in items:
                if is_first:
                    first_token_cost = time.time() - start_time
                    is_first = False
                    metadata["first_token_cost_ms"] = first_token_cost * 1000
                metadata["prompt_tokens"] = prompt_tokens
                out_count += 1
                yield sub_req_id, text, metadata, finish_status
                if finish_status.is_finished():
                    unfinished -= 1
                    if unfinished == 0:
                        total = time.time() - start_time
                        self.latest_success_infer_time_mark.set_value(int(time.time()))
                        if self.metric_client is not None:
                            m = self.metric_client
                            m.counter_inc("lightllm_request_success")
                            m.histogram_observe("lightllm_request_duration", total)
                            m.histogram_observe("lightllm_request_first_token_duration", first_token_cost or 0.0)
                            m.histogram_observe("lightllm_request_generated_tokens", out_count)
                            m.histogram_observe("lightllm_request_mean_time_per_token_duration",
                                                total / max(out_count, 1))
                        if self.args.detail_log:
                            print(f"req {group_req_id}: first_token {1e3 * (first_token_cost or 0):.1f} ms, total "
                                  f"{1e3 * total:.1f} ms, prompt {prompt_tokens}, out {out_count}, "
                                  f"prompt_cache_len {metadata.get('prompt_cache_len', 0)}", flush=True)
                        return

    def _prompt_logprobs_of(self, r) -> list:
        """One entry per prompt position: None for the first, then {token id: {"logprob", "rank", "decoded_token"}}
        with the prompt's own token (`prompt_logprobs` = 0) or the k most likely tokens and the prompt's own one
        (`prompt_logprobs` = k).  Reference: lightllm/server/core/objs/token_metadata.py:100-157."""
        tok = self.tokenizer

        def info(tid, lp, rank):
            try:
                text = tok.decode([tid], skip_special_tokens=False)
            except Exception:
                text = None
            return {"logprob": float(lp), "rank": rank, "decoded_token": text}

        meta = getattr(r, "shm_prompt_meta", None)
        k = (meta.arr.shape[1] - 1) // 2 if meta is not None else 0
        out = [None]
        for pos in range(1, r.input_len):
            tid = int(r.shm_prompt_ids.arr[pos])
            rank = int(meta.arr[pos, 0]) if meta is not None and meta.arr[pos, 0] > 0 else None
            entry = {}
            if k and rank is not None:
                for j in range(k):
                    entry[int(meta.arr[pos, 1 + j])] = info(int(meta.arr[pos, 1 + j]), meta.arr[pos, 1 + k + j], j + 1)
            entry[tid] = info(tid, r.shm_logprobs.arr[pos], rank)
            out.append(entry)
        return out

    async def abort(self, group_req_id: int) -> bool:
        st = self.req_id_to_out_inf.get(group_req_id)
        if st is None:
            return False
        for r in st.req_objs:
            r.is_aborted = True
        return True

    async def abort_by_master_id(self, master_req_id: int) -> bool:
        gid = self.master_id_to_local.get(master_req_id)
        return False if gid is None else await self.abort(gid)

    async def abort_all(self):
        for gid in list(self.req_id_to_out_inf):
            await self.abort(gid)

    # ------------------------------------------------------------------ background loops
    async def handle_loop(self):
        asyncio.create_task(self.recycle_resource_loop())
        while True:
            try:
                # the detokenizer's messages are wake-ups only; polling first (instead of cancelling a pending
                # receive after a timeout) never drops one in the middle of its delivery
                if await self.recv_from_detok.poll(50):
                    await self.recv_from_detok.recv_pyobj()
            except Exception:
                await asyncio.sleep(0.01)
            try:
                for st in list(self.req_id_to_out_inf.values()):
                    pulled = []
                    for r in st.req_objs:
                        q = r.out_tokens_queue
                        while not q.is_empty():
                            text, src_index, special, count = q.peek()
                            lp = float(r.shm_logprobs.arr[src_index])
                            tok_id = int(r.shm_prompt_ids.arr[src_index])
                            metadata = {"id": tok_id, "logprob": lp, "cumlogprob": float(r.cumlogprob),
                                        "special": special, "count_output_tokens": count,
                                        "prompt_cache_len": r.prompt_cache_len,
                                        "cpu_prompt_cache_len": r.cpu_prompt_cache_len,
                                        "disk_prompt_cache_len": r.disk_prompt_cache_len,
                                        "mtp_accepted_token_num": r.mtp_accepted_token_num}
                            q.pop_no_ret()
                            if r.finish_token_index == src_index and r.finish_status.is_finished():
                                fs = FinishStatus(r.finish_status.get_status())
                            elif r.stop_str_matched and r.stop_str_matched_token_index == src_index:
                                fs = FinishStatus(FinishStatus.FINISHED_STOP)
                            else:
                                fs = FinishStatus()
                            if r.request_id in st.finished:
                                continue
                            if fs.is_finished():
                                st.finished.add(r.request_id)
                                if r.sample_params.prompt_logprobs >= 0:
                                    metadata["prompt_token_ids"] = r.shm_prompt_ids.arr[: r.input_len].tolist()
                                    metadata["prompt_logprobs"] = self._prompt_logprobs_of(r)
                                if getattr(r, "shm_routed", None) is not None and r.routed_len > 0:
                                    from ...common.route_capture import encode

                                    metadata["routed_experts"] = encode(r.shm_routed.arr[:r.routed_len].copy())
                            pulled.append((r.request_id, text, metadata, fs))
                        # an aborted request is dropped by the detokenizer at once, so its last token may never
                        # arrive: once the detokenizer has let go of it and nothing is queued, the stream is ended
                        # here (a client may still be listening, e.g. after /abort_request)
                        if r.is_aborted and r.can_released_mark and q.is_empty() and r.request_id not in st.finished:
                            st.finished.add(r.request_id)
                            pulled.append((r.request_id, "", {"id": -1, "logprob": 0.0, "cumlogprob": float(r.cumlogprob),
                                                              "special": True, "count_output_tokens": r.shm_cur_output_len,
                                                              "prompt_cache_len": r.prompt_cache_len,
                                                              "cpu_prompt_cache_len": r.cpu_prompt_cache_len,
                                                              "disk_prompt_cache_len": r.disk_prompt_cache_len,
                                                              "mtp_accepted_token_num": r.mtp_accepted_token_num},
                                           FinishStatus(FinishStatus.FINISHED_ABORTED)))
                    if pulled:
                        async with st.lock:
                            st.out_token_info_list.extend(pulled)
                            st.event.set()
            except Exception:
                import traceback

                traceback.print_exc()

    async def recycle_resource_loop(self):
        while True:
            await asyncio.sleep(0.02)
            for gid, st in list(self.req_id_to_out_inf.items()):
                # only after every sub-request's final item has been handed to its stream
                if st.can_release() and all(r.request_id in st.finished for r in st.req_objs):
                    del self.req_id_to_out_inf[gid]
                    for r in st.req_objs:
                        r.release_shm_arrays(unlink=True)
                        idx = r.index_in_shm_mem
                        await self.shm_req_manager.async_put_back_req_obj(r)
                        await self.shm_req_manager.async_release_req_index(idx)

    # ------------------------------------------------------------------ control plane
    async def profiler_cmd(self, what: str):
        await self.send_to_router.send_pyobj(ProfilerCmd(what))

    async def flush_cache(self):
        await self.send_to_router.send_pyobj(FlushCacheCmd())

    async def rl_op(self, op: str, payload=None):
        await self.send_to_router.send_pyobj(RLCmd(op, payload))
