"""Seeded random weights: in memory, or written as a model folder.

The reference has no random-weights mode (its tests inject hash maps,
vllm-oxide crates/vllm-oxide/src/layers/linear.rs:187-190).  Every tensor gets its own
generator, seeded from (seed, tensor name), so the values do not depend on the order in
which tensors are made.  Scheme "fan_in": embeddings N(0,1), matrices N(0, 1/fan_in);
scheme "0.02": both N(0, 0.02^2); norm weights 1 + 0.1*N(0,1) in either.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Iterable

import torch

from .loader import TensorSpec, kept_dtype
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec: TensorSpec, seed: int, scheme: str, device, dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    x = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32)
    if spec.role == "norm":
        x = 1.0 + 0.1 * x
    elif spec.role == "bias":
        x = 0.02 * x
    elif scheme == "0.02":
        x = 0.02 * x
    elif scheme == "fan_in":
        if spec.role == "matrix":
            x = x / (float(spec.fan_in or spec.shape[-1]) ** 0.5)
    else:
        raise ValueError(f"unknown init scheme {scheme!r} (use 'fan_in' or '0.02')")
    return x.to(dtype)


def random_weights(specs: Iterable[TensorSpec], seed: int, scheme: str, device,
                   model_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """{name: tensor} in kept dtypes, generated on `device` (no file is written)."""
    return {s.name: random_tensor(s, seed, scheme, device, kept_dtype(s.role, model_dtype)) for s in specs}


def write_model_folder(folder: str, config_dict: dict, specs: Iterable[TensorSpec], seed: int,
                       scheme: str = "fan_in", store_dtype: torch.dtype = torch.bfloat16) -> None:
    """config.json and model.safetensors of a random model; every tensor stored in `store_dtype`."""
    from ..config.model_config import write_config_json
    os.makedirs(folder, exist_ok=True)
    tensors = {}
    for s in specs:
        dt = torch.int32 if s.role == "table" else store_dtype
        tensors[s.name] = random_tensor(s, seed, scheme, "cpu", dt)
    names = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}
    config_dict = dict(config_dict, torch_dtype=names.get(store_dtype, "bfloat16"))
    write_config_json(folder, config_dict)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
