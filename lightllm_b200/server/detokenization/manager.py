"""Detokenization process: turns the token ids the model ranks publish into text.

It learns about requests from the router (zmq), polls `candetoken_out_len` of every live
request, decodes incrementally, matches stop *strings* (stop token sequences are matched on the
rank), pushes (text, index, special, count) into the request's shm ring and wakes the HTTP
workers with a zmq PUB tick.  It is the last stage of the pipeline, so it also sets
`can_released_mark`.  Reference: lightllm/server/detokenization/manager.py:25-185.
"""
from __future__ import annotations

import time
import traceback
from typing import Dict

import zmq

from ..core.objs.io_objs import GroupReqIndexes
from ..core.objs.shm_req_manager import ShmReqManager
from ..core.objs.start_args import StartArgs, set_env_start_args
from ..tokenizer import get_tokenizer
from .decode import DecodeReq, decode_token


class DeTokenizationManager:
    def __init__(self, args: StartArgs):
        from ..router.manager import zmq_addr

        self.args = args
        ctx = zmq.Context(2)
        self.recv_from_router = ctx.socket(zmq.PULL)
        self.recv_from_router.bind(zmq_addr(args, args.detokenization_port))
        self.pub_to_http = ctx.socket(zmq.PUB)
        self.pub_to_http.bind(zmq_addr(args, args.http_server_port))
        self.tokenizer = get_tokenizer(args.model_dir, args.tokenizer_mode, args.trust_remote_code, args.vocab_size)
        self.all_special_ids = set(getattr(self.tokenizer, "all_special_ids", []) or [])
        self.eos_ids = set(args.eos_ids or [])
        self.req_id_to_out: Dict[int, DecodeReq] = {}
        self.shm_req_manager = ShmReqManager(args.unique_server_name, args.running_max_req_size)
        self.running = True

    def _add_new_group_req_index(self, g: GroupReqIndexes):
        for idx in g.shm_req_indexes:
            r = self.shm_req_manager.get_req_obj_by_index(idx)
            r.link_prompt_ids_shm_array(self.args.unique_server_name)
            r.link_logprobs_shm_array(self.args.unique_server_name)
            self.req_id_to_out[r.request_id] = DecodeReq(r)

    def handle_loop(self):
        while self.running:
            try:
                for _ in range(64):
                    try:
                        msg = self.recv_from_router.recv_pyobj(zmq.NOBLOCK)
                    except zmq.ZMQError:
                        break
                    if isinstance(msg, GroupReqIndexes):
                        self._add_new_group_req_index(msg)
                    elif msg == "exit":
                        self.running = False
                busy = self.gen_token_out()
                self.remove_finished_reqs()
                if not busy:
                    time.sleep(0.002)
            except Exception:
                traceback.print_exc()
                time.sleep(0.01)

    def gen_token_out(self) -> bool:
        produced = False
        for d in self.req_id_to_out.values():
            r = d.req
            if r.stop_str_matched:
                continue
            while d.need_detoken() and not d.out_queue_is_full():
                tok, src_index = d.get_next_token_id_and_index()
                text = decode_token(self.tokenizer, d, tok, self.eos_ids)
                special = tok in self.all_special_ids
                if r.is_aborted and src_index == r.finish_token_index and r.finish_status.get_status() == 3:
                    # the place-holder token with which an aborted request is ended (the router writes one for a
                    # request that never ran): it carries no text
                    text, special = "", True
                count = len(d.output_ids)
                if d.stop_strs and d.stop_sequences_str_match():
                    # the ranks are told through the router; generation ends at this token
                    r.stop_str_matched_token_index = src_index
                    r.stop_str_matched = True
                r.out_tokens_queue.push(text, src_index, special, count)
                produced = True
                if r.stop_str_matched:
                    break
        if produced:
            self.pub_to_http.send_pyobj(None)
        return produced

    def remove_finished_reqs(self):
        done = [d for d in self.req_id_to_out.values() if d.can_set_release_mark()]
        for d in done:
            r = d.req
            r.can_released_mark = True
            del self.req_id_to_out[d.request_id]
            r.release_shm_arrays(unlink=False)
            self.shm_req_manager.put_back_req_obj(r)
        if done:
            self.pub_to_http.send_pyobj(None)


def start_detokenization_process(args_dict: dict, pipe_writer):
    from ...utils.process_utils import graceful_registry, set_proc_title, start_parent_check_thread

    args = StartArgs.from_dict(args_dict)
    set_env_start_args(args)
    set_proc_title(f"lightllm::{args.unique_server_name}::detokenization_server")
    graceful_registry("detokenization")
    start_parent_check_thread()
    try:
        mgr = DeTokenizationManager(args)
    except Exception:
        pipe_writer.send(traceback.format_exc())
        raise
    pipe_writer.send("init ok")
    mgr.handle_loop()
