"""Shared fixtures: tiny configurations, random model folders, the plain implementation."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _cfg(**kw):
    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", attention_bias=False)
    base.update(kw)
    return base


# Tiny configurations that differ in every size and option (A, B, C), and one whose sizes reach the kernels that
# serving sizes use (D: 64-wide heads for the TMA and tcgen05 attention kernels, widths that are multiples of 64
# for the weight-streaming product and its fused SiLU*up, a window in one layer, pages of 64 keys; E: 128-wide
# heads on pages of 16 keys).
TINY = {
    # all-keys attention, tied output, 4 query heads over 2 key/value heads
    "A": dict(config=_cfg(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                          intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                          max_position_embeddings=512, tie_word_embeddings=True),
              seed=0, block_size=16),
    # one key/value head, q width 192 != hidden 80, odd vocabulary, separate output matrix
    "B": dict(config=_cfg(num_hidden_layers=3, hidden_size=80, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
                          intermediate_size=160, vocab_size=331, rope_theta=1000000.0, rms_norm_eps=1e-5,
                          max_position_embeddings=1024, tie_word_embeddings=False),
              seed=1, block_size=32),
    # sliding window of 24 in the last two of four layers, head_dim 48, nothing a power of two
    "C": dict(config=_cfg(num_hidden_layers=4, hidden_size=96, num_attention_heads=3, num_key_value_heads=3, head_dim=48,
                          intermediate_size=200, vocab_size=517, rope_theta=500000.0, rms_norm_eps=3e-6,
                          max_position_embeddings=2048, tie_word_embeddings=False, use_sliding_window=True,
                          sliding_window=24, max_window_layers=2),
              seed=2, block_size=16),
    "D": dict(config=_cfg(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                          intermediate_size=192, vocab_size=400, rope_theta=10000.0, rms_norm_eps=1e-6,
                          max_position_embeddings=1024, tie_word_embeddings=False, use_sliding_window=True,
                          sliding_window=40, max_window_layers=1),
              seed=3, block_size=64),
    # 128-wide heads (two 64-column slices a tile) on pages of 16 keys (a tile is then copied in runs of 16 keys,
    # slice by slice), one key/value head for two query heads, tied output
    "E": dict(config=_cfg(num_hidden_layers=2, hidden_size=192, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                          intermediate_size=320, vocab_size=211, rope_theta=50000.0, rms_norm_eps=1e-5,
                          max_position_embeddings=512, tie_word_embeddings=True),
              seed=4, block_size=16),
}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """{name: folder} of the tiny random models, weights stored in float32 so that both dtypes start
    from the same numbers (bfloat16 runs round them)."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    out = {}
    for name, spec in TINY.items():
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_random_model_folder(folder, spec["config"], spec["seed"], "fan_in", torch.float32)
        out[name] = folder
    return out


@pytest.fixture(scope="session")
def plain_models(model_folders):
    """{name: (config dict, weights)} as the plain implementation reads them."""
    from plain import qwen3_plain
    return {name: qwen3_plain.read_folder(folder) for name, folder in model_folders.items()}


def tokens_for(name: str, n: int, salt: int = 0):
    g = torch.Generator().manual_seed(1000 * TINY[name]["seed"] + salt + 17)
    return torch.randint(0, TINY[name]["config"]["vocab_size"], (n,), generator=g).tolist()
