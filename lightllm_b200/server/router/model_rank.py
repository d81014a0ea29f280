"""Model-rank process: one per GPU.  Builds the model and its `ModelBackend`, then self-drives:
it polls the router's shm mailbox for commands (new requests, aborts, stop-string hits, profiler
and RL operations) and runs prefill / decode steps; results go straight into the shm requests.

Ranks of one tensor-parallel group must apply mailbox commands at the same step boundary.  The
mailbox carries a generation counter; before each step the ranks of a node agree on the newest
generation all of them have seen with a one-integer MIN all-reduce on the host (gloo) group, so
no GPU collective and no device sync sits in the polling loop.

Reference: lightllm/server/router/model_infer/model_rpc.py:56-238 (process entry, init_model)
and mode_backend/base_backend.py:473-606 (_try_read_new_reqs, _init_reqs).
"""
from __future__ import annotations

import os
import time
import traceback
from typing import Optional

import torch

from ..core.objs.atomic_lock import SharedArray
from ..core.objs.io_objs import AbortedReqCmd, FlushCacheCmd, NewReqsCmd, ProfilerCmd, RLCmd, StopStrMatchedReqCmd
from ..core.objs.shm_objs_io_buffer import ShmObjsIOBuffer
from ..core.objs.shm_req_manager import ShmReqManager
from ..core.objs.start_args import StartArgs, set_env_start_args


class ExitCmd:
    pass


def _state_slots(args) -> int:
    """Recurrent-state snapshot slots of hybrid models (`--linear_att_cache_size`); none when the prefix cache is
    off.  Models without linear-attention layers ignore the number."""
    if getattr(args, "disable_dynamic_prompt_cache", False):
        return 0
    n = getattr(args, "linear_att_cache_size", None)
    return int(n) if n else 32


def _kv_type(args):
    """`--llm_kv_type`: None / "None" keep the model dtype; "int8kv" selects the quantised pool."""
    k = getattr(args, "llm_kv_type", None)
    return None if k in (None, "None", "none", "") else k


def _mtp_modules(args) -> int:
    """Draft modules to build: one per step for the vanilla modes, one reused module for the eagle modes."""
    if not getattr(args, "mtp_mode", None):
        return 0
    return 1 if str(args.mtp_mode).startswith("eagle") else max(1, int(args.mtp_step))


def _publishes(args, ps) -> bool:
    """The rank of a replica that writes tokens and finish states into its node's shared request objects: the
    replica's first rank, and, when a tensor-parallel replica spans nodes, its first rank on every node (each node has
    its own request objects, HTTP server and detokenizer)."""
    per_node = max(1, args.tp // args.nnodes)
    return ps.tp_rank % min(ps.tp_size, per_node) == 0


def _build_model_and_backend(args: StartArgs, ps):
    from ...engine.backend import BackendArgs, ModelBackend
    from ...models.base import load_config
    from ...models.registry import get_model

    cfg = getattr(args, "_config_override", None) or load_config(args.model_dir)
    fused = None
    if ps.tp_size > 1 and ps.device.type == "cuda" and not args.disable_symm_mem_allreduce:
        try:
            from ...parallel.fused import FusedTP

            hidden = cfg.get("hidden_size") or (cfg.get("text_config") or {}).get("hidden_size")
            fused = FusedTP(ps, max_tokens=args.batch_max_tokens, hidden=int(hidden))
            if not fused.self_test():   # all ranks see the same answer
                print(f"[rank {ps.global_rank}] fused tensor-parallel reduction failed its start-up probe: "
                      "falling back to NCCL", flush=True)
                fused.close()
                fused = None
        except Exception:
            fused = None
    model = get_model(cfg, model_dir=args.model_dir, pstate=ps, data_type=args.data_type,
                      max_total_token_num=args.max_total_token_num, mem_fraction=args.mem_fraction,
                      max_req_num=args.running_max_req_size, max_seq_length=args.max_req_total_len + 8,
                      batch_max_tokens=args.batch_max_tokens, disable_cudagraph=args.disable_cudagraph,
                      graph_max_batch_size=min(args.graph_max_batch_size, args.running_max_req_size),
                      graph_split_batch_size=args.graph_split_batch_size,
                      graph_grow_step_size=args.graph_grow_step_size,
                      graph_max_len_in_batch=args.graph_max_len_in_batch or None, tp_fused=fused,
                      enable_ep_moe=args.enable_ep_moe, quant_type=args.quant_type,
                      quant_cfg=getattr(args, "quant_cfg", None), expert_dtype=getattr(args, "expert_dtype", None),
                      extra_kv_layers=_mtp_modules(args), kv_type=_kv_type(args),
                      state_snapshot_slots=_state_slots(args),
                      linear_att_ssm_data_type=getattr(args, "linear_att_ssm_data_type", "float32"),
                      kv_quant_calibration_config_path=getattr(args, "kv_quant_calibration_config_path", None),
                      tpsp_mix_mode=bool(getattr(args, "enable_tpsp_mix_mode", False)),
                      ep_redundancy_expert_config_path=getattr(args, "ep_redundancy_expert_config_path", None),
                      auto_update_redundancy_expert=bool(getattr(args, "auto_update_redundancy_expert", False)),
                      enable_return_routed_experts=bool(getattr(args, "enable_return_routed_experts", False)),
                      enable_dp_prefill_balance=bool(getattr(args, "enable_dp_prefill_balance", False)),
                      kv_quant_group_size=getattr(args, "llm_kv_quant_group_size", 8),
                      enable_fused_shared_experts=bool(getattr(args, "enable_fused_shared_experts", False)))
    if fused is not None:   # prompt passes as two micro-batches with copy-engine reductions
        from ...parallel import ce as _ce

        _ce.attach(model, ps, args.batch_max_tokens)
    eos = args.eos_ids or args.eos_id or cfg.get("eos_token_id") or []
    eos = tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
    bargs = BackendArgs(batch_max_tokens=args.batch_max_tokens, chunked_prefill_size=args.chunked_prefill_size,
                        disable_chunked_prefill=args.disable_chunked_prefill,
                        router_max_wait_tokens=args.router_max_wait_tokens,
                        disable_aggressive_schedule=args.disable_aggressive_schedule,
                        disable_dynamic_prompt_cache=args.disable_dynamic_prompt_cache, eos_ids=eos,
                        max_req_total_len=args.max_req_total_len,
                        return_all_prompt_logprobs=args.enable_prompt_logprobs,
                        cpu_cache_bytes=int(args.cpu_cache_storage_size * (1 << 30)) if args.enable_cpu_cache else 0,
                        cpu_cache_page_tokens=args.cpu_cache_token_page_size,
                        disk_cache_dir=args.disk_cache_dir if args.enable_disk_cache else None,
                        disk_cache_bytes=int(args.disk_cache_storage_size * (1 << 30)) if args.enable_disk_cache else 0,
                        linear_att_hash_page_size=int(getattr(args, "linear_att_hash_page_size", 512) or 512),
                        state_host_cache_bytes=int(args.cpu_cache_storage_size * (1 << 30)) if (
                            args.enable_cpu_cache and not getattr(args, "disable_linear_att_small_page_cpu_cache", False))
                        else 0)
    from ...engine.mode_backends import select_backend_class

    backend_cls = select_backend_class(args)
    kw = {}
    if args.run_mode == "prefill":
        kw = dict(tp_rank=ps.tp_rank, page_tokens=args.pd_kv_page_size,
                  cpu_group=ps.cpu_group if ps.dp_size == 1 else None, tp_size=ps.tp_size)
    elif args.run_mode == "decode":
        on_done = None
        if ps.tp_rank == 0 and args.pd_kv_status_port:
            import zmq

            sock = zmq.Context.instance().socket(zmq.PUSH)
            sock.connect(f"tcp://127.0.0.1:{args.pd_kv_status_port}")
            on_done = lambda gid, ok: sock.send_pyobj((gid, ok))  # noqa: E731
        # a rank receives KV pages on pd_kv_port + its global rank (replica j, tensor-parallel rank t: j * tp + t)
        kw = dict(tp_rank=ps.global_rank if ps.dp_size > 1 else ps.tp_rank,
                  host=args.host if args.host not in ("localhost",) else "127.0.0.1",
                  kv_port=args.pd_kv_port, page_tokens=args.pd_kv_page_size, page_num=args.pd_kv_page_num,
                  cpu_group=ps.cpu_group if ps.dp_size == 1 else None, tp_size=ps.tp_size, on_kv_done=on_done)
    elif backend_cls.__name__ in ("TokenHealingBackend", "XgrammarBackend", "OutlinesConstraintBackend"):
        from ..tokenizer import get_tokenizer

        kw = dict(tokenizer=get_tokenizer(args.model_dir, args.tokenizer_mode, args.trust_remote_code, args.vocab_size))
    if _mtp_modules(args):
        from ...engine.mtp_backend import MTPBackend
        from ...models.mtp import build_mtp_modules

        draft_dir = args.mtp_draft_model_dir
        if isinstance(draft_dir, (list, tuple)):
            draft_dir = draft_dir[0] if draft_dir else None
        drafts = build_mtp_modules(model, _mtp_modules(args), model_dir=draft_dir or args.model_dir)
        mkw = {}
        if ps.dp_size > 1:       # lock-step data parallelism: every replica runs the same passes per round
            assert args.run_mode not in ("prefill", "decode"), \
                "speculative decoding on P/D nodes with --dp > 1 is not supported"
            from ...engine.mtp_backend import DPMTPBackend as MTPBackend  # noqa: F811
        elif args.run_mode in ("prefill", "decode"):
            from ...engine.mode_backends import pd_mtp_classes

            MTPBackend = pd_mtp_classes()[0 if args.run_mode == "prefill" else 1]  # noqa: F811
            mkw = kw
        backend = MTPBackend(model, bargs, draft_models=drafts, mtp_step=args.mtp_step,
                             is_master_in_dp=_publishes(args, ps), **mkw)
    else:
        backend = backend_cls(model, bargs, is_master_in_dp=_publishes(args, ps), **kw)
    if getattr(args, "enable_multimodal", False):
        from ..embed_cache.cache import EmbedArena
        from ..embed_cache.manager import arena_name, arena_rows

        width = getattr(model, "embed_row_width", model.hidden)
        model.embed_arena = EmbedArena(arena_name(args), arena_rows(args, width), width, create=False)
    return model, backend


class ModelRankLoop:
    def __init__(self, args: StartArgs, rank: int, ps, model, backend):
        self.args = args
        self.rank = rank
        self.ps = ps
        self.model = model
        self.backend = backend
        name = args.unique_server_name
        self.node_world = args.tp // args.nnodes
        self.mailbox = ShmObjsIOBuffer(f"{name}_router_to_ranks", self.node_world)
        self.shm_req_manager = ShmReqManager(name, args.running_max_req_size)
        # [rank, (free tokens, radix unreferenced tokens, running reqs)] read by the router
        self.load_arr = SharedArray(f"{name}_rank_load", (args.tp, 4), "int64")
        self.last_gen = self.mailbox.generation()
        self.running = True
        self.profiler = None
        self.dp_index = ps.dp_rank
        self.prefix_fetch = bool(getattr(args, "enable_dp_prompt_cache_fetch", False)) and ps.dp_size > 1 and \
            args.nnodes == 1 and backend.radix_cache is not None

    def _agree_generation(self) -> int:
        g = self.mailbox.generation()
        if self.ps.world_size == 1 or self.ps.cpu_group is None:
            return g
        t = torch.tensor([g], dtype=torch.int64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN, group=self.ps.cpu_group)
        return int(t.item())

    def _handle(self, cmd):
        b = self.backend
        if isinstance(cmd, NewReqsCmd):
            mine = []
            if self.prefix_fetch:     # copy prefixes another replica has cached before the requests are admitted
                b.fetch_prefixes([(dp_index, self._peek_prompt(shm_index)) for _, shm_index, _, dp_index in cmd.reqs])
            for req_id, shm_index, mm_params, dp_index in cmd.reqs:
                if self.ps.dp_size > 1 and dp_index != self.dp_index:
                    continue
                r = self.shm_req_manager.get_req_obj_by_index(shm_index)
                r.link_prompt_ids_shm_array(self.args.unique_server_name)
                r.link_logprobs_shm_array(self.args.unique_server_name)
                if r.sample_params.prompt_logprobs >= 0 and self.args.enable_prompt_logprobs:
                    r.link_prompt_meta_shm_array(self.args.unique_server_name)
                rc = getattr(self.model, "route_capture", None)
                if rc is not None:
                    r.link_routed_shm_array(self.args.unique_server_name, rc.num_layers, rc.top_k, rc.np_dtype)
                r._mm_params = mm_params
                mine.append(r)
            if mine:
                b.add_reqs(mine)
        elif isinstance(cmd, AbortedReqCmd):
            b.abort(cmd.req_id)
        elif isinstance(cmd, StopStrMatchedReqCmd):
            b.stop_str_matched(cmd.req_id)
        elif isinstance(cmd, ProfilerCmd):
            self._profiler_cmd(cmd.cmd)
        elif isinstance(cmd, FlushCacheCmd):
            if b.radix_cache is not None and not b.has_work():
                b.radix_cache.clear_tree_nodes()
        elif isinstance(cmd, RLCmd):
            from ...engine.rl_ops import handle_rl_cmd

            handle_rl_cmd(self, cmd)
        elif isinstance(cmd, ExitCmd):
            self.running = False

    def _peek_prompt(self, shm_index: int):
        """Prompt token ids of a request that may belong to another replica (read through a short-lived link)."""
        r = self.shm_req_manager.get_req_obj_by_index(shm_index)
        try:
            r.link_prompt_ids_shm_array(self.args.unique_server_name)
            ids = r.shm_prompt_ids.arr[: r.input_len].copy()
            r.shm_prompt_ids.close_shm(unlink=None)
            r.shm_prompt_ids = None
            return ids
        finally:
            self.shm_req_manager.put_back_req_obj(r)

    def _profiler_cmd(self, what: str):
        from ...utils.profiler import ProcessProfiler

        if self.profiler is None:
            self.profiler = ProcessProfiler(self.args.enable_profiling or "torch_profiler", f"rank{self.rank}")
        self.profiler.cmd(what)

    def _read_mailbox(self):
        g = self._agree_generation()
        if g == self.last_gen:
            return
        cmds = self.mailbox.read_obj()
        self.last_gen = g
        self.mailbox.sub_state()
        for c in cmds:
            self._handle(c)

    def _publish_load(self):
        b = self.backend
        row = self.load_arr.arr[self.ps.global_rank]
        row[0] = self.model.mem_manager.can_use_mem_size
        row[1] = b.radix_cache.unreferenced_tokens_num() if b.radix_cache is not None else 0
        row[2] = len(b.ctx.requests)
        row[3] = int(time.time())

    def run(self):
        idle_sleep = 0.001
        while self.running:
            self._read_mailbox()
            if hasattr(self.backend, "poll_kv"):
                self.backend.poll_kv()
            if self.backend.has_work():
                res = self.backend.step()
                for ir in res["finished"]:
                    ir.shm_req.release_shm_arrays(unlink=False)
                    self.shm_req_manager.put_back_req_obj(ir.shm_req)
            else:
                time.sleep(idle_sleep)
            self._publish_load()


def model_rank_main(args_dict: dict, rank: int, pipe, config_override: Optional[dict] = None):
    """Process entry (spawned by the router)."""
    try:
        from ...parallel import dist as pdist
        from ...utils.process_utils import set_proc_title, start_parent_check_thread

        args = StartArgs.from_dict(args_dict)
        set_env_start_args(args)
        set_proc_title(f"lightllm::{args.unique_server_name}::model_infer:RANK{rank}")
        start_parent_check_thread()
        use_cuda = torch.cuda.is_available() and args.hardware_platform == "cuda" and \
            os.environ.get("LLB_FORCE_CPU", "0") != "1"
        node_world = args.tp // args.nnodes
        local_rank = rank % node_world
        device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
        if not use_cuda and args.tp > 1:
            # CPU ranks (tests: also the "nodes") of one host share its cores: without a limit every rank's math
            # library spins on all of them
            torch.set_num_threads(max(1, (os.cpu_count() or 2) // args.tp))
        ps = pdist.init_distributed(args.tp, rank, dp=args.dp, nnodes=args.nnodes, node_rank=args.node_rank,
                                    host=args.nccl_host, port=args.nccl_port, device=device,
                                    config_server=(args.config_server_host, args.config_server_port)
                                    if getattr(args, "use_config_server_to_init_nccl", False) else None)
        if config_override is not None:
            args._config_override = config_override
        model, backend = _build_model_and_backend(args, ps)
        loop = ModelRankLoop(args, rank, ps, model, backend)
        pipe.send(("init ok", model.max_total_token_num))
    except Exception:
        pipe.send(("init failed", traceback.format_exc()))
        return
    try:
        loop.run()
    except Exception:
        traceback.print_exc()
        os._exit(-1)
