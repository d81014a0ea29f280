"""Redundant experts under expert parallelism (`--ep_redundancy_expert_config_path`, `--auto_update_redundancy_expert`).

With data-parallel attention and expert-parallel MoE every rank owns E / world experts.  A rank may hold R more
experts as copies of experts that live elsewhere; a token of THIS rank routed to one of them is served by the copy,
so it neither crosses NVLink nor queues on the owner.  Physical expert ids are rank x (E / world + R) + local index;
every rank rewrites the router's ids through its own table (`ops.moe.count_remap`, which also keeps the per-expert
hit counter), and the exchange and the grouped GEMMs work in the physical id space unchanged.

Static placement comes from the JSON file the reference uses: {"redundancy_expert_num": R, "<layer>": [ids],
"default": [ids]}.  With `--auto_update_redundancy_expert` a manager on every rank re-places its copies from its own
counters every LLB_REDUNDANCY_EXPERT_UPDATE_INTERVAL seconds: pick the R most-hit experts that are not local, read
them from the checkpoint on a thread, then between two steps copy them into the slots and switch the table.  Slots,
table and counters keep their addresses, so captured CUDA graphs stay valid.  Rank 0 also writes the world's R
most-hit experts per layer to `redundancy_expert_config.json` as a static file for the next start.

Reference: lightllm/server/router/model_infer/mode_backend/redundancy_expert_manager.py:1-158,
lightllm/common/basemodel/layer_weights/meta_weights/fused_moe/ep_redundancy.py,
lightllm/utils/envs_utils.py:99-146 (file format).
"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Dict, List, Optional

import torch


class RedundancyConfig:
    def __init__(self, num: int = 0, per_layer: Optional[Dict[str, List[int]]] = None, default: Optional[List[int]] = None):
        self.num = int(num)
        self.per_layer = per_layer or {}
        self.default = list(default or [])
        if self.num:
            for k, ids in list(self.per_layer.items()) + [("default", self.default)]:
                if ids and len(ids) != self.num:
                    raise ValueError(f"redundancy expert config: entry {k!r} lists {len(ids)} experts, "
                                     f"redundancy_expert_num is {self.num}")

    @classmethod
    def load(cls, path: Optional[str]) -> "RedundancyConfig":
        if not path:
            return cls()
        with open(path) as f:
            cfg = json.load(f)
        num = int(cfg.get("redundancy_expert_num", 0))
        layers = {k: [int(e) for e in v] for k, v in cfg.items() if k not in ("redundancy_expert_num", "default")}
        return cls(num, layers, [int(e) for e in cfg.get("default", [])])

    def ids(self, layer: int) -> List[int]:
        if not self.num:
            return []
        ids = self.per_layer.get(str(layer), self.default)
        return list(ids) if ids else list(range(self.num))


def physical_table(num_experts: int, world: int, rank: int, red_ids: List[int]) -> torch.Tensor:
    """table[e] = physical id of expert e as seen from `rank`."""
    el, R = num_experts // world, len(red_ids)
    e = torch.arange(num_experts, dtype=torch.int64)
    table = (e // el) * (el + R) + e % el
    for j, rid in enumerate(red_ids):
        if not 0 <= rid < num_experts:
            raise ValueError(f"redundant expert id {rid} is outside 0..{num_experts - 1}")
        if rid // el != rank:               # a copy of an expert this rank owns anyway would only waste the slot
            table[rid] = rank * (el + R) + el + j
    return table.to(torch.int32)


def write_expert_slot(stacked, slot: int, value) -> None:
    """Copies one expert's matrix into row block `slot` of a stacked expert tensor (bf16 [E, N, K], or block-scaled
    e4m3 `Fp8Experts` with a one-expert `Fp8Weight` as value)."""
    if type(stacked).__name__ == "Fp8Experts":
        N = stacked.shape[1]
        g = stacked.w.ws_rows
        stacked.w.q.view(torch.uint8)[slot * N:(slot + 1) * N].copy_(value.q.view(torch.uint8), non_blocking=True)
        stacked.w.scale[slot * (N // g):(slot + 1) * (N // g)].copy_(value.scale, non_blocking=True)
    else:
        stacked[slot].copy_(value, non_blocking=True)


class RedundancyExpertManager:
    CHECK, LOADING, COMMIT = range(3)

    def __init__(self, model, interval_s: Optional[float] = None, max_updates: Optional[int] = None,
                 out_path: str = "./redundancy_expert_config.json"):
        self.model = model
        self.layers = [lw for lw in model.layers if getattr(lw, "ep_table", None) is not None]
        def env(name, default):      # the reference's spelling of the variable is honoured too
            return os.environ.get("LLB_" + name, os.environ.get("LIGHTLLM_" + name, default))

        self.interval = float(env("REDUNDANCY_EXPERT_UPDATE_INTERVAL", 30 * 60)) if interval_s is None else interval_s
        self.max_updates = int(env("REDUNDANCY_EXPERT_UPDATE_MAX_LOAD_COUNT", 1)) if max_updates is None \
            else max_updates
        self.updates = 0
        self.state = self.CHECK
        self.last = time.time()
        self.thread: Optional[threading.Thread] = None
        self.staged: Dict[int, tuple] = {}
        self.error: Optional[BaseException] = None
        self.out_path = out_path
        for lw in self.layers:
            lw.ep_counter.zero_()

    # ------------------------------------------------------------------
    def step(self) -> bool:
        """Call between two model steps (no kernel of this rank in flight reads the slots).  True when new copies
        were committed in this call."""
        if self.updates >= self.max_updates or not self.layers:
            return False
        if self.state == self.CHECK:
            if time.time() - self.last >= self.interval:
                self.last = time.time()
                plan = self._choose()
                self.thread = threading.Thread(target=self._load, args=(plan,), daemon=True)
                self.thread.start()
                self.state = self.LOADING
        elif self.state == self.LOADING:
            if not self.thread.is_alive():
                self.thread = None
                if self.error is not None:     # keep serving with the old placement
                    print(f"[redundancy] reading the new copies failed: {self.error!r}", flush=True)
                    self.error, self.staged, self.state = None, {}, self.CHECK
                    self.updates += 1
                else:
                    self.state = self.COMMIT
        elif self.state == self.COMMIT:
            self._commit()
            self.state = self.CHECK
            self.updates += 1
            return True
        return False

    def _choose(self) -> Dict[int, List[int]]:
        m = self.model
        world, rank = m.ps.world_size, m.ps.global_rank
        plan, static = {}, {}
        for lw in self.layers:
            cnt = lw.ep_counter.detach().cpu().to(torch.int64)
            lw.ep_counter.zero_()
            R = lw.ep_red_num
            static[str(lw.ep_layer)] = [int(e) for e in torch.argsort(cnt, stable=True)[-R:]]
            el = cnt.numel() // world
            cnt[rank * el:(rank + 1) * el] = -1          # never a copy of an expert this rank owns
            plan[lw.ep_layer] = [int(e) for e in torch.argsort(cnt, stable=True)[-R:]]
        if rank == 0 and self.out_path:
            try:
                R = self.layers[0].ep_red_num
                with open(self.out_path, "w") as f:
                    json.dump({"redundancy_expert_num": R, "default": list(range(R)), **static}, f, indent=1)
            except OSError as e:
                print(f"[redundancy] could not write {self.out_path}: {e}", flush=True)
        return plan

    def _load(self, plan):
        try:
            for lw in self.layers:
                ids = plan[lw.ep_layer]
                self.staged[lw.ep_layer] = (ids, [lw.ep_read_expert(e) for e in ids])
        except BaseException as e:   # surfaced by step()
            self.error = e

    def _commit(self):
        m = self.model
        world, rank = m.ps.world_size, m.ps.global_rank
        for lw in self.layers:
            ids, mats = self.staged.pop(lw.ep_layer)
            el = lw.ep_table.numel() // world
            for j, (w13, w2) in enumerate(mats):
                write_expert_slot(lw.w13, el + j, w13)
                write_expert_slot(lw.w2, el + j, w2)
            lw.ep_table.copy_(physical_table(lw.ep_table.numel(), world, rank, ids))
            lw.ep_red_ids = ids
        if m.device.type == "cuda":
            torch.cuda.synchronize(m.device)
