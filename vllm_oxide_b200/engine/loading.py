"""From a model folder (or a configuration and a seed) to a model on the device."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config.model_config import read_config_json
from ..models.causal_lm import CausalLM
from ..models.registry import resolve
from ..weights.loader import kept_dtype, load_checked
from ..weights.random_init import random_tensor, random_weights, write_model_folder

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def resolve_dtype(name: Optional[str]) -> torch.dtype:
    name = name or "bfloat16"
    if name not in DTYPES:
        raise ValueError(f"dtype {name!r} is not supported: 'bfloat16' (serving) or 'float32' (true 32-bit)")
    return DTYPES[name]


def load_model(folder: str, dtype: torch.dtype, device) -> Tuple[object, CausalLM]:
    """The model named by `folder`/config.json with the weights of its safetensors files."""
    config_dict = read_config_json(folder)
    cfg, plan = resolve(config_dict, where=f"{folder}/config.json")
    model = CausalLM(plan, dtype, device)
    model.unexpected_tensors = []      # names the folder holds and the model does not use (ignored, with a warning)
    model.load(load_checked(folder, model.tensor_specs(), dtype, device, unexpected=model.unexpected_tensors))
    return cfg, model


def random_model(config_dict: dict, seed: int, dtype: torch.dtype, device, scheme: str = "fan_in",
                 draw_on: Optional[str] = None):
    """The model of `config_dict` with seeded random weights.  They are drawn directly on the device (fast at any
    size; the device's generator) unless `draw_on="cpu"`: then every tensor is drawn by the host's generator, which
    gives the values that `write_random_model_folder` stores for the same seed, and moved to the device."""
    cfg, plan = resolve(config_dict, where="config")
    model = CausalLM(plan, dtype, device)
    if draw_on is None or torch.device(draw_on) == torch.device(device):
        model.load(random_weights(model.tensor_specs(), seed, scheme, device, dtype))
    else:
        model.load({s.name: random_tensor(s, seed, scheme, draw_on, torch.float32).to(
            device=device, dtype=kept_dtype(s.role, dtype)) for s in model.tensor_specs()})
    return cfg, model


def write_random_model_folder(folder: str, config_dict: dict, seed: int, scheme: str = "fan_in",
                              store_dtype: torch.dtype = torch.bfloat16) -> None:
    """config.json and model.safetensors of a random model of `config_dict`."""
    cfg, plan = resolve(config_dict, where="config")
    specs = CausalLM(plan, torch.float32, "cpu").tensor_specs()
    out = dict(config_dict)
    if hasattr(cfg, "to_dict"):
        out = {**cfg.to_dict(), **{k: v for k, v in config_dict.items() if k not in ("torch_dtype", "dtype")}}
    write_model_folder(folder, out, specs, seed, scheme, store_dtype)
