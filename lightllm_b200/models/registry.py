"""Model registry keyed on HF ``config.json: model_type`` (reference: lightllm/models/registry.py)."""
from __future__ import annotations

from typing import Callable, Dict, Optional

_REGISTRY: Dict[str, list] = {}


def register_model(*model_types: str, condition: Optional[Callable[[dict], bool]] = None, is_multimodal=False):
    def deco(cls):
        for mt in model_types:
            _REGISTRY.setdefault(mt, []).append((condition, cls, is_multimodal))
        return cls

    return deco


def get_model_class(config: dict):
    from . import _load_all  # noqa: F401  (imports every model module once)

    mt = config.get("model_type")
    cands = _REGISTRY.get(mt)
    if not cands:
        raise ValueError(f"unsupported model_type {mt!r}; known: {sorted(_REGISTRY)}")
    # conditional entries first
    for cond, cls, _ in cands:
        if cond is not None and cond(config):
            return cls
    for cond, cls, _ in cands:
        if cond is None:
            return cls
    raise ValueError(f"no registered variant of {mt!r} accepts this config")


def is_multimodal(config: dict) -> bool:
    from . import _load_all  # noqa: F401

    cands = _REGISTRY.get(config.get("model_type"), [])
    for cond, _, mm in cands:   # the variant that `get_model_class` would pick
        if cond is not None and cond(config):
            return bool(mm)
    return any(mm for cond, _, mm in cands if cond is None)


def supported_model_types():
    from . import _load_all  # noqa: F401

    return sorted(_REGISTRY)


def get_model(config: dict, **kvargs):
    return get_model_class(config)(config, **kvargs)
