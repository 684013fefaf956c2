"""Typed model configuration, read from the architecture's own config.json keys.

`Qwen3Config` holds exactly what a Qwen3 (dense) config.json gives; no size of the model
lives anywhere else in the package.  The keys and their defaults follow the reference's
`Qwen3Config` (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:26-58) with three
deliberate differences, each an error instead of a silent change of model:

* `attention_bias` defaults to False (the reference defaults it to true and thereby drops
  q_norm/k_norm, qwen3.rs:52-54,124-139; every published Qwen3 config says false);
* `hidden_act` must be "silu" (the reference requires the key and never reads it, :40);
* `rope_scaling` must be absent or null; the window keys (`use_sliding_window`,
  `sliding_window`, `max_window_layers`), which the reference ignores, are honoured.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong type, or asks for something unsupported."""


_DTYPE_NAMES = {
    # crates/vllm-oxide/src/config.rs:90-105
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float16": "float16", "fp16": "float16", "half": "float16",
    "float32": "float32", "fp32": "float32", "float": "float32",
    "float64": "float64", "fp64": "float64", "double": "float64",
}


def _need(d: dict, key: str, typ, where: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
        if v <= 0:
            raise ConfigError(f"{where}: '{key}' must be positive, got {v}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    eos_token_id: Optional[int] = None

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "Qwen3Config":
        hidden = _need(d, "hidden_size", int, where)
        heads = _need(d, "num_attention_heads", int, where)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{where}: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads  # qwen3.rs:48-51
        elif isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim <= 0:
            raise ConfigError(f"{where}: 'head_dim' must be a positive integer, got {head_dim!r}")
        kv = _need(d, "num_key_value_heads", int, where)
        if heads % kv:
            raise ConfigError(f"{where}: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv}")
        if head_dim % 2:
            raise ConfigError(f"{where}: head_dim {head_dim} must be even for rotate-half position encoding")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: hidden_act {act!r} is not supported (only 'silu')")
        if d.get("rope_scaling") is not None:
            raise ConfigError(f"{where}: rope_scaling {d['rope_scaling']!r} is not supported")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        use_window = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        if use_window:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"{where}: use_sliding_window needs a positive 'sliding_window', got {window!r}")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        return cls(
            hidden_size=hidden,
            num_hidden_layers=_need(d, "num_hidden_layers", int, where),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=_need(d, "intermediate_size", int, where),
            vocab_size=_need(d, "vocab_size", int, where),
            rms_norm_eps=_need(d, "rms_norm_eps", float, where),
            rope_theta=float(d.get("rope_theta", 1_000_000.0)),  # qwen3.rs:22-24
            max_position_embeddings=_need(d, "max_position_embeddings", int, where),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),  # qwen3.rs:55-57
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=act,
            torch_dtype=_DTYPE_NAMES[dtype],
            use_sliding_window=use_window,
            sliding_window=int(window) if use_window else None,
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            eos_token_id=eos,
        )

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen3"
        if not self.use_sliding_window:
            d["sliding_window"] = None
        return d

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer's attention, None for all keys: with `use_sliding_window`,
        layers from `max_window_layers` on see the last `sliding_window` positions."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in the model folder")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(folder: str, config_dict: dict) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_dict, f, indent=1, sort_keys=True)
