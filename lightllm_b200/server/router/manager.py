"""Router process: admission scheduling for one node.

Receives `GroupReqIndexes` from the HTTP worker(s) over zmq, keeps the waiting queue(s), and every
`schedule_time_interval` decides which waiting requests join the running batch (Past-Future
estimate against the KV pool size published by the model ranks).  Admitted requests, aborts and
stop-string hits are handed to the model ranks through the shm mailbox; the ranks drive prefill /
decode themselves and the router never sits on the token path.

Reference: lightllm/server/router/manager.py:45-512.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import pickle
import socket
import time
import traceback
from typing import Dict, List, Optional

import zmq

from ..core.objs.atomic_lock import SharedArray, SharedInt
from ..core.objs.io_objs import (AbortedReqCmd, FlushCacheCmd, GroupReqIndexes, NewReqsCmd, ProfilerCmd, RLCmd,
                                 StopStrMatchedReqCmd)
from ..core.objs.req import Req
from ..core.objs.shm_objs_io_buffer import ShmObjsIOBuffer
from ..core.objs.shm_req_manager import ShmReqManager
from ..core.objs.start_args import StartArgs, set_env_start_args
from .model_rank import ExitCmd, model_rank_main
from .req_queue import Batch, RouterStatics, build_req_queue
from .token_load import TokenLoad


def zmq_addr(args, port) -> str:
    if args.zmq_mode.startswith("ipc"):
        return f"{args.zmq_mode}{args.unique_server_name}_{port}"
    return f"tcp://127.0.0.1:{port}"


class RouterManager:
    MULTINODE_WAIT_S = float(os.environ.get("LLB_MULTINODE_WAIT_S", 30.0))

    def __init__(self, args: StartArgs, config_override: Optional[dict] = None):
        self.args = args
        self.name = args.unique_server_name
        self.config_override = config_override
        self.node_world = args.tp // args.nnodes
        self.dp_size_in_node = max(1, args.dp // args.nnodes)
        ctx = zmq.Context(2)
        self.recv_from_http = ctx.socket(zmq.PULL)
        self.recv_from_http.bind(zmq_addr(args, args.router_port))
        self.send_to_detok = ctx.socket(zmq.PUSH)
        self.send_to_detok.connect(zmq_addr(args, args.detokenization_port))
        self.shm_req_manager = ShmReqManager(self.name, args.running_max_req_size)
        self.mailbox = ShmObjsIOBuffer(f"{self.name}_router_to_ranks", self.node_world)
        self.load_arr = SharedArray(f"{self.name}_rank_load", (args.tp, 4), "int64")
        self.shm_max_total_token_num = SharedInt(f"{self.name}_max_total_token_num")
        self.token_load = TokenLoad(f"{self.name}_token_load", self.dp_size_in_node)
        self.statics = RouterStatics()
        self.running_batch: Optional[Batch] = None
        self.pending_cmds: List = []
        self.rank_procs: List[mp.Process] = []
        self.batch_id = 0
        self.req_queue = None
        self.max_total_token_num = 0
        self._last_load_refresh = 0.0
        self.metrics = None
        self.mn_sync = None     # server/router/multinode_sync.py when --nnodes > 1 and --dp 1
        self._mn_dropped = set()  # group ids of waiting requests that node 0 dropped (client gone)
        self._exit_flushed = False

    # ------------------------------------------------------------------ start-up
    def wait_to_model_ready(self):
        ctx = mp.get_context("spawn")
        pipes = []
        first = self.args.node_rank * self.node_world
        for r in range(first, first + self.node_world):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=model_rank_main, args=(self.args.to_dict(), r, child, self.config_override))
            p.start()
            self.rank_procs.append(p)
            pipes.append(parent)
        totals = []
        for p, pipe in zip(self.rank_procs, pipes):
            while not pipe.poll(0.5):
                if not p.is_alive():
                    raise RuntimeError(f"model rank died during start-up (exit code {p.exitcode})")
            status, payload = pipe.recv()
            if status != "init ok":
                raise RuntimeError(f"model rank failed to start:\n{payload}")
            totals.append(int(payload))
        self.max_total_token_num = min(totals)
        self.args.max_total_token_num = self.max_total_token_num
        self.shm_max_total_token_num.set_value(self.max_total_token_num)
        self.req_queue = build_req_queue(self.args, self.max_total_token_num, self.dp_size_in_node, self.statics)
        if self.args.nnodes > 1 and self.args.dp == 1:
            self._init_multinode_sync()

    def _init_multinode_sync(self):
        """A gloo group of the routers (one per node) on `--multinode_router_gloo_port` of node 0's address; the
        pool size every router plans with is the smallest one any node measured."""
        import datetime

        import torch
        import torch.distributed as dist

        from .multinode_sync import MultiNodeRouterSync

        a = self.args
        dist.init_process_group("gloo", init_method=f"tcp://{a.nccl_host}:{a.multinode_router_gloo_port}",
                                rank=a.node_rank, world_size=a.nnodes, timeout=datetime.timedelta(minutes=30))
        t = torch.tensor([self.max_total_token_num], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if int(t) != self.max_total_token_num:
            self.max_total_token_num = int(t)
            self.args.max_total_token_num = self.max_total_token_num
            self.shm_max_total_token_num.set_value(self.max_total_token_num)
            self.req_queue = build_req_queue(a, self.max_total_token_num, self.dp_size_in_node, self.statics)
        self.mn_sync = MultiNodeRouterSync(None, a.node_rank, a.nnodes)

    # ------------------------------------------------------------------ loop pieces
    def _recv_new_reqs(self, limit: int = 256):
        got = 0
        while got < limit:
            try:
                msg = self.recv_from_http.recv_pyobj(zmq.NOBLOCK)
            except zmq.ZMQError:
                break
            got += 1
            if isinstance(msg, GroupReqIndexes):
                self._add_req(msg)
            elif isinstance(msg, (ProfilerCmd, FlushCacheCmd, RLCmd)):
                self.pending_cmds.append(msg)
            elif isinstance(msg, ExitCmd):
                self.pending_cmds.append(msg)
        return got

    def _add_req(self, g: GroupReqIndexes):
        reqs = []
        for idx in g.shm_req_indexes:
            r = self.shm_req_manager.get_req_obj_by_index(idx)
            r._mm_params = g.multimodal_params
            if r.group_req_id in self._mn_dropped:      # node 0 dropped it before it got here
                self._mn_dropped.discard(r.group_req_id)
                r.is_aborted = True
            reqs.append(r)
        self.req_queue.extend(reqs)
        self.send_to_detok.send_pyobj(g, protocol=pickle.HIGHEST_PROTOCOL)

    def _usage_ratio(self) -> float:
        """Pool usage seen by the ranks of the first replica (free + evictable radix tokens count as free)."""
        row = self.load_arr.arr[self.args.node_rank * self.node_world]
        free = int(row[0]) + int(row[1])
        if self.max_total_token_num <= 0:
            return 0.0
        return max(0.0, 1.0 - free / self.max_total_token_num)

    def _schedule(self):
        ratio = self._usage_ratio()
        if hasattr(self.req_queue, "set_usage"):
            self.req_queue.set_usage([ratio] * self.dp_size_in_node)
        else:
            self.req_queue.cur_token_usage_ratio = ratio
        paused = self.running_batch is not None and any(r.is_paused for r in self.running_batch.reqs)
        if paused:
            return None
        self.batch_id += 1
        return self.req_queue.generate_new_batch(self.running_batch, self.batch_id)

    def _abort_and_stop_cmds(self):
        cmds = []
        if self.running_batch is not None:
            for r in self.running_batch.reqs:
                if r.is_aborted and not getattr(r, "_abort_sent", False):
                    r._abort_sent = True
                    cmds.append(AbortedReqCmd(r.request_id))
                if r.stop_str_matched and not getattr(r, "_stop_sent", False):
                    r._stop_sent = True
                    cmds.append(StopStrMatchedReqCmd(r.request_id))
        return cmds

    def _new_reqs_cmd(self, batch: Batch):
        return NewReqsCmd([(r.request_id, r.index_in_shm_mem, getattr(r, "_mm_params", None),
                            r.sample_params.suggested_dp_index) for r in batch.reqs])

    def _round_multinode(self):
        """One scheduling round of a multi-node tensor-parallel deployment (see router/multinode_sync.py): node 0
        decides, every node admits the same groups in the same order and writes the same message to its ranks."""
        q, sync = self.req_queue, self.mn_sync
        waiting = list(dict.fromkeys(r.group_req_id for r in q.waiting_req_list if not r.is_aborted))
        all_free, allowed = sync.gather(waiting, self.mailbox.is_empty())
        plan = None
        if sync.is_master:
            # a request that some node never received (its relay failed there, e.g. no free request slot) would
            # block everything behind it in arrival order for ever: after a while the master gives it up
            now = time.time()
            for r in q.waiting_req_list:
                if not r.is_aborted and r.group_req_id not in allowed and now - r.recv_time > self.MULTINODE_WAIT_S:
                    print(f"[router] request {r.group_req_id} did not arrive on every node within "
                          f"{self.MULTINODE_WAIT_S:.0f} s: dropped", flush=True)
                    r.is_aborted = True
            chosen, cmds = [], []
            if all_free:
                cmds, self.pending_cmds = list(self.pending_cmds), []
                paused = self.running_batch is not None and any(r.is_paused for r in self.running_batch.reqs)
                if not paused:
                    ratio = self._usage_ratio()
                    if hasattr(q, "set_usage"):
                        q.set_usage([ratio] * self.dp_size_in_node)
                    b = q.generate_new_batch(self.running_batch, self.batch_id + 1, allowed_groups=allowed)
                    if b is not None:
                        q.waiting_req_list = b.reqs + q.waiting_req_list      # take() below removes them again
                        chosen = list(dict.fromkeys(r.group_req_id for r in b.reqs))
                cmds += self._abort_and_stop_cmds()
            plan = (chosen, cmds, sorted(self._mn_dropped))
            self._mn_dropped.clear()
        chosen, cmds, dropped = sync.broadcast(plan)
        if not sync.is_master and dropped:
            self._mn_dropped.update(dropped)
            for r in q.waiting_req_list:
                if r.group_req_id in self._mn_dropped:
                    r.is_aborted = True
        self.batch_id += 1
        new_batch = q.take(chosen, self.batch_id)
        if new_batch is not None:
            cmds = cmds + [self._new_reqs_cmd(new_batch)]
        if cmds:
            self.mailbox.write_obj(cmds)
            self.mailbox.set_ready()
            if any(isinstance(c, ExitCmd) for c in cmds):
                self._exit_flushed = True
        if new_batch is not None:
            if self.running_batch is None:
                self.running_batch = new_batch
            else:
                self.running_batch.merge(new_batch)

    def _flush_mailbox(self, new_batch: Optional[Batch]):
        """Writes everything pending (new batch, aborts, stop hits, control commands) as one message."""
        if not self.mailbox.is_empty():
            return False
        cmds = list(self.pending_cmds)
        self.pending_cmds = []
        if new_batch is not None:
            cmds.append(self._new_reqs_cmd(new_batch))
        cmds += self._abort_and_stop_cmds()
        if not cmds:
            return True
        self.mailbox.write_obj(cmds)
        self.mailbox.set_ready()
        return True

    def _release_waiting_aborted(self):
        for r in self.req_queue.pop_aborted():
            # never reached a rank: the router finishes it so that detokenizer / HTTP can drain
            r.link_prompt_ids_shm_array(self.name)
            r.link_logprobs_shm_array(self.name)
            r.shm_prompt_ids.arr[r.input_len] = 0
            r.shm_cur_output_len = 1
            r.finish_token_index = r.input_len
            r.finish_status.set_status(3)
            r.candetoken_out_len = 1
            r.shm_infer_released = True
            r.release_shm_arrays()
            self.shm_req_manager.put_back_req_obj(r)

    def _step(self):
        self._recv_new_reqs()
        if self.mn_sync is not None and self.mn_sync.is_master:
            self._mn_dropped.update(r.group_req_id for r in self.req_queue.waiting_req_list if r.is_aborted)
        self._release_waiting_aborted()
        new_batch = None
        if self.mn_sync is not None:
            self._round_multinode()
        elif self.mailbox.is_empty():
            new_batch = self._schedule()
            if self._flush_mailbox(new_batch) and new_batch is not None:
                if self.running_batch is None:
                    self.running_batch = new_batch
                else:
                    self.running_batch.merge(new_batch)
        if self.running_batch is not None:
            done = self.running_batch.filter_out_finished_req(self.shm_req_manager)
            for r in done:
                self.statics.update(r.shm_cur_output_len)
            if self.running_batch.is_clear():
                self.running_batch = None
        now = time.time()
        if now - self._last_load_refresh > 1.0:
            self._last_load_refresh = now
            loads = self.req_queue.calcu_batch_token_load(self.running_batch)
            if not isinstance(loads, list):
                loads = [loads]
            for i, (peak, cur) in enumerate(loads):
                self.token_load.set(i, cur, peak, self._usage_ratio())
            if self.metrics is not None:
                self.metrics.gauge_set("lightllm_batch_current_size", len(self.running_batch) if self.running_batch else 0)
                self.metrics.gauge_set("lightllm_queue_size", self.req_queue.get_wait_req_num())

    def loop_for_fwd(self):
        interval = self.args.schedule_time_interval
        exiting = False
        while not exiting:
            t0 = time.time()
            self._step()
            if self.mn_sync is not None:
                exiting = self._exit_flushed
            elif any(isinstance(c, ExitCmd) for c in self.pending_cmds):
                while not self._flush_mailbox(None):
                    time.sleep(0.001)
                exiting = True
            for p in self.rank_procs:
                if not p.is_alive():
                    raise RuntimeError(f"model rank exited with code {p.exitcode}")
            dt = time.time() - t0
            if dt < interval:
                # poll the socket while waiting so that bursts are picked up promptly
                if self.recv_from_http.poll(int((interval - dt) * 1000)):
                    pass
        for p in self.rank_procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()


def start_router_process(args_dict: dict, config_override, pipe_writer):
    from ...utils.process_utils import graceful_registry, set_proc_title, start_parent_check_thread

    args = StartArgs.from_dict(args_dict)
    set_env_start_args(args)
    set_proc_title(f"lightllm::{args.unique_server_name}::router")
    graceful_registry("router")
    start_parent_check_thread()
    try:
        router = RouterManager(args, config_override)
        router.wait_to_model_ready()
    except Exception:
        pipe_writer.send(traceback.format_exc())
        raise
    pipe_writer.send("init ok")
    try:
        router.loop_for_fwd()
    except Exception:
        traceback.print_exc()
        for p in router.rank_procs:
            if p.is_alive():
                p.kill()
        raise
