"""Weights by name: shard resolution, one error for everything that is wrong, random folders."""
import json
import os

import pytest
import torch

from conftest import TINY
from vllm_oxide_b200.engine.loading import write_random_model_folder
from vllm_oxide_b200.models import CausalLM, resolve
from vllm_oxide_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_checked, resolve_shards,
                                     write_safetensors)


def specs_of(name):
    _, plan = resolve(TINY[name]["config"])
    return CausalLM(plan, torch.float32, "cpu").tensor_specs()


def test_names_and_shapes_are_the_checkpoints():
    s = {x.name: x.shape for x in specs_of("B")}
    assert s["model.layers.2.self_attn.q_proj.weight"] == (192, 80)
    assert s["model.layers.0.self_attn.k_proj.weight"] == (32, 80)
    assert s["model.layers.1.self_attn.o_proj.weight"] == (80, 192)
    assert s["model.layers.1.self_attn.q_norm.weight"] == (32,)
    assert s["model.layers.0.mlp.gate_proj.weight"] == (160, 80) and s["model.layers.0.mlp.down_proj.weight"] == (80, 160)
    assert s["lm_head.weight"] == (331, 80) and s["model.norm.weight"] == (80,)
    assert "lm_head.weight" not in {x.name for x in specs_of("A")}      # tied


def test_roundtrip_and_kept_dtypes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model_folder(folder, TINY["A"]["config"], 0, "fan_in", torch.bfloat16)
    specs = specs_of("A")
    w = load_checked(folder, specs, torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert w["model.norm.weight"].dtype == torch.float32                 # norm weights are kept in 32-bit
    w32 = load_checked(folder, specs, torch.float32, "cpu")
    assert torch.equal(w32["model.embed_tokens.weight"], w["model.embed_tokens.weight"].float())
    again = str(tmp_path / "m2")
    write_random_model_folder(again, TINY["A"]["config"], 0, "fan_in", torch.bfloat16)
    w2 = load_checked(again, specs, torch.bfloat16, "cpu")
    assert all(torch.equal(w[k], w2[k]) for k in w)                      # the seed decides the values
    other = str(tmp_path / "m3")
    write_random_model_folder(other, TINY["A"]["config"], 5, "fan_in", torch.bfloat16)
    assert not torch.equal(load_checked(other, specs, torch.bfloat16, "cpu")["model.norm.weight"], w["model.norm.weight"])
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["architectures"] == ["Qwen3ForCausalLM"]


def test_init_scheme_statistics(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model_folder(folder, TINY["B"]["config"], 1, "fan_in", torch.float32)
    w = load_checked(folder, specs_of("B"), torch.float32, "cpu")
    assert abs(w["model.embed_tokens.weight"].std() - 1.0) < 0.05
    assert abs(w["model.layers.0.mlp.down_proj.weight"].std() - 160 ** -0.5) < 0.01
    assert abs(w["model.layers.0.input_layernorm.weight"].mean() - 1.0) < 0.05


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model_folder(folder, TINY["A"]["config"], 0, "fan_in", torch.float32)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)       # should be [32, 64]
    tensors["model.layers.7.extra.weight"] = torch.zeros(3)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_checked(folder, specs_of("A"), torch.float32, "cpu")
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.7.extra.weight" in msg
    assert "model.layers.0.self_attn.k_proj.weight expected [32, 64] found [16, 64]" in msg
    assert sorted(e.value.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.7.extra.weight"]


def test_tensors_the_model_does_not_use_are_a_warning_not_an_error(tmp_path):
    """A folder with tied output that also stores lm_head.weight and a rotary buffer loads (the reference never reads
    them, crates/vllm-oxide/src/models/qwen3.rs:322-331); the names are kept for the caller; strict refuses them."""
    from vllm_oxide_b200.weights.loader import UnexpectedTensorsWarning
    folder = str(tmp_path / "m")
    write_random_model_folder(folder, TINY["A"]["config"], 0, "fan_in", torch.float32)       # A: tied output
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    plain = load_checked(folder, specs_of("A"), torch.float32, "cpu")
    tensors["lm_head.weight"] = torch.randn(256, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    seen = []
    with pytest.warns(UnexpectedTensorsWarning, match="lm_head.weight"):
        w = load_checked(folder, specs_of("A"), torch.float32, "cpu", unexpected=seen)
    assert seen == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert set(w) == set(plain) and all(torch.equal(w[k], plain[k]) for k in w)
    with pytest.raises(WeightsError) as e:
        load_checked(folder, specs_of("A"), torch.float32, "cpu", strict=True)
    assert e.value.unexpected == seen and not e.value.missing and not e.value.wrong_shape


def test_shard_resolution(tmp_path):
    d = tmp_path
    with pytest.raises(SafetensorsError, match="no weights found"):
        resolve_shards(str(d))
    write_safetensors(str(d / "b.safetensors"), {"x": torch.zeros(2)})
    write_safetensors(str(d / "a.safetensors"), {"y": torch.ones(3)})
    assert [os.path.basename(p) for p in resolve_shards(str(d))] == ["a.safetensors", "b.safetensors"]
    write_safetensors(str(d / "model.safetensors"), {"z": torch.ones(1)})
    assert [os.path.basename(p) for p in resolve_shards(str(d))] == ["model.safetensors"]
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "b.safetensors", "q": "c.safetensors"}}))
    with pytest.raises(SafetensorsError, match="partial"):
        resolve_shards(str(d))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "b.safetensors", "y": "a.safetensors"}}))
    assert [os.path.basename(p) for p in resolve_shards(str(d))] == ["a.safetensors", "b.safetensors"]


def test_truncated_file_is_refused(tmp_path):
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, {"x": torch.arange(100, dtype=torch.float32)})
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:-40])
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(p)
    open(p, "wb").write(blob[:6])
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)


def test_merged_rows_order():
    """q rows, then k rows, then v rows; gate rows, then up rows (crates/vllm-oxide/src/layers/linear.rs:211-239,306-326)."""
    from vllm_oxide_b200.parts import PartSpec, build_part
    att = build_part("mixer", PartSpec("attention", dict(hidden_size=8, num_heads=2, num_kv_heads=1, head_dim=16, eps=1e-6,
                                                           qkv_bias=True, qk_norm=False, window=None, position="p", prefix="a.")),
                     positions={"p": None}, dtype=torch.float32, device="cpu")
    t = {s.name: torch.full(s.shape, float(i + 1)) for i, s in enumerate(att.tensor_specs())}
    att.load(t)
    assert att.wqkv.shape == (64, 8)
    assert att.wqkv[0, 0] == 1 and att.wqkv[32, 0] == 2 and att.wqkv[48, 0] == 3
    assert att.bqkv[0] == 5 and att.bqkv[32] == 6 and att.bqkv[48] == 7
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=8, intermediate_size=12, prefix="m.")))
    t = {s.name: torch.full(s.shape, float(i + 1)) for i, s in enumerate(ffn.tensor_specs())}
    ffn.load(t)
    assert ffn.wgu.shape == (24, 8) and ffn.wgu[0, 0] == 1 and ffn.wgu[12, 0] == 2 and not ffn.interleaved
    # an intermediate size that is a multiple of 8 is stored as groups of 8 gate rows + the 8 up rows of the same outputs
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=4, intermediate_size=16, prefix="m.")))
    t = {s.name: torch.arange(s.shape[0], dtype=torch.float32)[:, None].expand(s.shape) + 100 * i
         for i, s in enumerate(ffn.tensor_specs())}
    ffn.load(t)
    assert ffn.interleaved and ffn.wgu[:, 0].tolist() == ([0, 1, 2, 3, 4, 5, 6, 7] + [100 + r for r in range(8)]
                                                           + [8 + r for r in range(8)] + [108 + r for r in range(8)])
