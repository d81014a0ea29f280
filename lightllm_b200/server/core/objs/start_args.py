"""Typed launch arguments shared by every process of a server.

`StartArgs` mirrors the CLI flags plus derived fields; the launcher serialises it as JSON into
the environment (LIGHTLLM_START_ARGS) so that spawned processes and HTTP workers read the same
values (reference: lightllm/server/core/objs/start_args_type.py, lightllm/utils/envs_utils.py:35-50).
"""
from __future__ import annotations

import json
import os
from types import SimpleNamespace
from typing import Any, Dict

from ...api_cli import FLAGS

ENV_KEY = "LIGHTLLM_START_ARGS"

# fields derived by the launcher (not CLI flags)
DERIVED_DEFAULTS: Dict[str, Any] = {
    "router_port": None, "detokenization_port": None, "http_server_port": None, "visual_port": None,
    "audio_port": None, "cache_port": None, "metric_port": None, "multi_level_kv_cache_port": None,
    "pd_node_id": -1, "pd_kv_port": None, "pd_kv_status_port": None, "pd_p_allowed_port_min": 20000, "pd_p_allowed_port_max": 30000,
    "pd_decode_rpyc_port": None, "child_ips": None, "enable_multimodal": False, "enable_multimodal_audio": False,
    "unique_server_name": None, "cpu_kv_cache_shm_id": None, "weight_version": "default",
    "model_rpc_ports": None, "vocab_size": None, "eos_ids": None,
}


class StartArgs(SimpleNamespace):
    """Attribute bag with every flag of `api_cli.FLAGS` plus `DERIVED_DEFAULTS`."""

    @classmethod
    def defaults(cls) -> "StartArgs":
        d = {}
        for spec in FLAGS:
            d[spec[0].lstrip("-")] = spec[2]
        d.update(DERIVED_DEFAULTS)
        return cls(**d)

    @classmethod
    def from_namespace(cls, ns) -> "StartArgs":
        a = cls.defaults()
        for k, v in vars(ns).items():
            setattr(a, k, v)
        return a

    @classmethod
    def from_dict(cls, d: dict) -> "StartArgs":
        a = cls.defaults()
        for k, v in d.items():
            setattr(a, k, v)
        return a

    def to_dict(self) -> dict:
        return dict(vars(self))


def set_env_start_args(args) -> None:
    d = args.to_dict() if isinstance(args, StartArgs) else dict(vars(args))
    os.environ[ENV_KEY] = json.dumps(d, default=str)


_cached = None


def get_env_start_args() -> StartArgs:
    global _cached
    raw = os.environ.get(ENV_KEY)
    if raw is None:
        return StartArgs.defaults()
    if _cached is None or _cached[0] != raw:
        _cached = (raw, StartArgs.from_dict(json.loads(raw)))
    return _cached[1]


def get_unique_server_name() -> str:
    a = get_env_start_args()
    return a.unique_server_name or os.environ.get("LIGHTLLM_UNIQUE_SERVICE_NAME_ID", "llb")
