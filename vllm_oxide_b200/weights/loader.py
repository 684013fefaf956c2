"""Weights by tensor name, checked against what the model's parts declare.

Every part of a model lists the tensors it needs as `TensorSpec`s (checkpoint name, shape,
role).  `load_checked` compares the whole list with the files of a model folder and
raises ONE `WeightsError` that names every missing tensor, every unexpected tensor and
every tensor of the wrong shape.  The reference reads by name without a remap table
(vllm-oxide, crates/vllm-oxide/src/loader.rs:105-119) but leaves q/k/v shapes unchecked
(crates/vllm-oxide/src/layers/linear.rs:111-117); here nothing is unchecked.

A missing tensor or a wrong shape is always an error.  Tensors that the model does not ask
for are not, when nothing else is wrong: the reference never looks at them (a checkpoint with
tied output that also stores lm_head.weight loads there, crates/vllm-oxide/src/models/qwen3.rs:322-331;
so does one with rotary inv_freq buffers).  They are reported with an `UnexpectedTensorsWarning`,
kept in the list the caller passes as `unexpected`, and never read; `strict=True` makes them an
error too.

Kept dtypes: matrices and embeddings in the model dtype (bfloat16 when serving, float32
on the true 32-bit path); norm weights always in float32, so a norm weight stored in
32-bit stays so; integer tensors as int32.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, resolve_shards


@dataclass(frozen=True)
class TensorSpec:
    name: str                 # checkpoint name, e.g. model.layers.0.self_attn.q_proj.weight
    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix" | "embedding" | "norm" | "bias" | "table" (integer)
    fan_in: Optional[int] = None


class WeightsError(ValueError):
    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], other: List[str] = ()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"{where}: the weights do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        lines.extend(other)
        super().__init__("\n".join(lines))


class UnexpectedTensorsWarning(UserWarning):
    """The model folder holds tensors that the model does not use (they are ignored)."""


def kept_dtype(role: str, model_dtype: torch.dtype) -> torch.dtype:
    if role == "norm":
        return torch.float32
    if role == "table":
        return torch.int32
    return model_dtype


def check_specs(where: str, specs: Iterable[TensorSpec], found: Dict[str, tuple], strict: bool = False) -> List[str]:
    """Raises one `WeightsError` for missing tensors and wrong shapes (it lists the unexpected ones as well);
    returns the names of the unexpected tensors when they are all that is amiss (`strict`: they are an error too)."""
    specs = list(specs)
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in found]
    unexpected = sorted(n for n in found if n not in wanted)
    wrong = [(n, tuple(s.shape), tuple(found[n])) for n, s in wanted.items()
             if n in found and tuple(found[n]) != tuple(s.shape)]
    if missing or wrong or (strict and unexpected):
        raise WeightsError(where, missing, unexpected, wrong)
    return unexpected


def load_checked(folder: str, specs: Iterable[TensorSpec], model_dtype: torch.dtype, device, *,
                 strict: bool = False, unexpected: Optional[List[str]] = None) -> Dict[str, torch.Tensor]:
    """All tensors named by `specs`, on `device`, in their kept dtypes.  Tensors of the folder that no spec names
    are left unread: their names are appended to `unexpected` (if given) and a warning names them."""
    specs = list(specs)
    files = [SafetensorsFile(p) for p in resolve_shards(folder)]
    where_of: Dict[str, SafetensorsFile] = {}
    for f in files:
        for n in f.names():
            where_of[n] = f
    extra = check_specs(folder, specs, {n: f.shape(n) for n, f in where_of.items()}, strict)
    if extra:
        if unexpected is not None:
            unexpected.extend(extra)
        shown = ", ".join(extra[:8]) + (f", ... ({len(extra)} in all)" if len(extra) > 8 else "")
        warnings.warn(f"{folder}: {len(extra)} tensor(s) that the model does not use were ignored: {shown}",
                      UnexpectedTensorsWarning, stacklevel=2)
    out = {}
    for s in specs:
        t = where_of[s.name].tensor(s.name)
        if s.role == "table" and t.dtype.is_floating_point:
            raise WeightsError(folder, [], [], [], [f"  tensor {s.name} must be an integer table, found {t.dtype}"])
        out[s.name] = t.to(device=device, dtype=kept_dtype(s.role, model_dtype), copy=True)
    return out
