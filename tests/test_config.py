"""Typed configuration and the architecture registry."""
import json

import pytest

from conftest import TINY
from vllm_oxide_b200.config import ConfigError, EngineOptions, Qwen3Config, read_config_json
from vllm_oxide_b200.models import resolve, supported_architectures


def test_reads_every_size_from_config():
    c = Qwen3Config.from_dict(TINY["B"]["config"])
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (80, 3, 6, 1, 32)
    assert (c.intermediate_size, c.vocab_size, c.rms_norm_eps, c.rope_theta) == (160, 331, 1e-5, 1e6)
    assert c.max_position_embeddings == 1024 and c.tie_word_embeddings is False


def test_defaults_follow_the_reference():
    d = dict(TINY["A"]["config"])
    for k in ("head_dim", "rope_theta", "tie_word_embeddings", "attention_bias"):
        d.pop(k, None)
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 64 // 4            # hidden / heads
    assert c.rope_theta == 1_000_000.0
    assert c.tie_word_embeddings is False and c.attention_bias is False


def test_published_shape_of_a_real_config_parses():
    d = {"architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643,
         "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 1024, "initializer_range": 0.02,
         "intermediate_size": 3072, "max_position_embeddings": 40960, "max_window_layers": 28, "model_type": "qwen3",
         "num_attention_heads": 16, "num_hidden_layers": 28, "num_key_value_heads": 8, "rms_norm_eps": 1e-06,
         "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": True,
         "torch_dtype": "bfloat16", "use_cache": True, "use_sliding_window": False, "vocab_size": 151936}
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 128 and c.num_attention_heads * c.head_dim == 2048 != c.hidden_size
    assert c.eos_token_id == 151645 and c.layer_window(27) is None


@pytest.mark.parametrize("change, word", [
    ({"hidden_size": None}, "hidden_size"), ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"torch_dtype": "int8"}, "torch_dtype"), ({"vocab_size": -4}, "positive"), ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"), ({"rms_norm_eps": "x"}, "number"),
])
def test_bad_configs_are_refused(change, word):
    d = dict(TINY["A"]["config"])
    d.update(change)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_window_layers():
    c = Qwen3Config.from_dict(TINY["C"]["config"])
    assert [c.layer_window(i) for i in range(4)] == [None, None, 24, 24]


def test_registry_by_architecture_name(tmp_path):
    cfg, plan = resolve(TINY["A"]["config"])
    assert plan.architecture == "Qwen3ForCausalLM" and len(plan.layers) == 2 and plan.lm_head_name is None
    assert [s.layer for s in plan.order] == [0, 1]
    with pytest.raises(ConfigError, match="not supported.*Qwen3ForCausalLM"):
        resolve({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve({})
    assert "Qwen3ForCausalLM" in supported_architectures()
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_plan_chooses_parts_layer_by_layer():
    _, plan = resolve(TINY["C"]["config"])
    windows = [l.params["mixer"].params["window"] for l in plan.layers]
    assert windows == [None, None, 24, 24]
    assert plan.layers[0].params["mixer"].kind == "attention" and plan.layers[0].params["feed_forward"].kind == "swiglu"


def test_engine_options_defaults_and_checks():
    o = EngineOptions()
    assert (o.max_num_batched_tokens, o.max_num_seqs, o.max_model_len, o.gpu_memory_utilization) == (16384, 512, 4096, 0.9)
    o.validate()
    with pytest.raises(ValueError):
        EngineOptions(block_size=24).validate()
    with pytest.raises(ValueError):
        EngineOptions(dtype="float16").validate()


def test_decode_attention_split_counts():
    """How many blocks share the keys of a (request, kv head) in decode attention: what fits the GPU at once, at least
    two tiles of 64 keys each, a cluster (at most 8) unless few requests with long contexts make a second kernel pay."""
    from vllm_oxide_b200.parts.attention import decode_splits
    assert decode_splits(1, 8, 100, 148) == 1 and decode_splits(1, 8, 300, 148) == 2
    assert decode_splits(1, 8, 2304, 148) == 8 and decode_splits(8, 8, 2304, 148) == 4 and decode_splits(64, 8, 2304, 148) == 1
    assert decode_splits(1, 8, 40960, 148) == 32 and decode_splits(2, 8, 32768, 148) == 16 and decode_splits(3, 8, 32768, 148) == 12
    assert decode_splits(1, 8, 8192, 148) == 16 and decode_splits(1, 16, 32768, 148) == 16
    assert decode_splits(4, 8, 16384, 148) == 8          # 9 would fit: not enough to leave the cluster for
    assert decode_splits(8, 8, 32768, 148) == 4
    for requests in (1, 2, 3, 5, 8, 13, 40, 300):
        for keys in (1, 63, 64, 65, 1000, 8191, 8192, 100000):
            s = decode_splits(requests, 4, keys, 148)
            assert 1 <= s <= 32 and (s == 1 or 2 * s <= -(-keys // 64))
