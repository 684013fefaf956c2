"""One registry from the architecture's name (config.json `architectures[0]`) to its model.

As in the reference (vllm-oxide, crates/vllm-oxide/src/models/registry.rs:10-51) an unknown name
is an error that lists the supported ones.  An entry is (typed configuration class, plan function).
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from ..config.model_config import ConfigError, Qwen3Config
from .plan import ModelPlan
from .qwen3 import qwen3_plan

_ARCHITECTURES: Dict[str, Tuple[Callable[[dict], object], Callable[[object], ModelPlan]]] = {}


def register_architecture(name: str, config_from_dict: Callable[[dict], object],
                          plan_fn: Callable[[object], ModelPlan]) -> None:
    _ARCHITECTURES[name] = (config_from_dict, plan_fn)


def supported_architectures():
    return sorted(_ARCHITECTURES)


def resolve(config_dict: dict, where: str = "config.json"):
    """(typed config, plan) for a parsed config.json."""
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' must be a non-empty list of names")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"{where}: architecture {name!r} is not supported; supported: {supported_architectures()}")
    config_from_dict, plan_fn = _ARCHITECTURES[name]
    cfg = config_from_dict(config_dict)
    return cfg, plan_fn(cfg)


register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_plan)
