"""The plain implementation against closed forms (the reference's own unit-test vectors)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from plain import sampler_plain as S


def test_add_then_norm():
    # crates/vllm-oxide/src/layers/rmsnorm.rs:168-185: [3,0,0] + [0,4,0], weight 1, eps 1e-12
    y, r = P.add_rms_norm(torch.tensor([3.0, 0, 0]), torch.tensor([0.0, 4, 0]), torch.ones(3), 1e-12, torch.float32)
    assert r.tolist() == [3.0, 4.0, 0.0]
    rms = math.sqrt(25.0 / 3.0)
    assert torch.allclose(y, torch.tensor([3 / rms, 4 / rms, 0.0]), atol=1e-6)


def test_norm_without_residual_returns_input():
    x = torch.tensor([1.0, 2.0, 3.0])
    _, r = P.add_rms_norm(x, None, torch.ones(3), 1e-6, torch.float32)
    assert r.tolist() == x.tolist()   # rmsnorm.rs:187-198


def test_weight_scales_output():
    # rmsnorm.rs:204-219: x=[3,4,0,0], w=[10,20,30,40] -> [12, 32, 0, 0]
    y, _ = P.add_rms_norm(torch.tensor([3.0, 4, 0, 0]), None, torch.tensor([10.0, 20, 30, 40]), 1e-12, torch.float32)
    assert torch.allclose(y, torch.tensor([12.0, 32.0, 0, 0]), atol=1e-5)


def test_bf16_norm_close_to_fp32():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 8, generator=g)
    ref, _ = P.add_rms_norm(x, None, torch.ones(8), 1e-6, torch.float32)
    got, _ = P.add_rms_norm(x.bfloat16(), None, torch.ones(8), 1e-6, torch.bfloat16)
    assert (ref - got.float()).abs().max() < 3e-2   # rmsnorm.rs:128-152


def test_rope_table_shape_and_position_zero():
    t = P.rope_table(8, 32, 10000.0)
    assert t.shape == (32, 8)                     # rope.rs:174-178
    q = torch.arange(1.0, 9.0).reshape(1, 1, 8)
    out = P.apply_rope(q, torch.tensor([0]), t, torch.float32)
    assert torch.allclose(out, q, atol=1e-6)      # rope.rs:207-228
    assert not torch.allclose(P.rope_table(8, 16, 1e6), P.rope_table(8, 16, 1e4))   # rope.rs:245-262


def test_rope_is_a_rotation_by_position_times_inv_freq():
    hd, theta = 8, 10000.0
    t = P.rope_table(hd, 16, theta)
    x = torch.zeros(1, 1, hd)
    x[0, 0, 1] = 1.0          # pair (1, 1 + hd/2)
    out = P.apply_rope(x, torch.tensor([3]), t, torch.float32)[0, 0]
    ang = 3.0 / theta ** (2 / hd)
    assert abs(out[1] - math.cos(ang)) < 1e-6 and abs(out[1 + hd // 2] - math.sin(ang)) < 1e-6


def test_silu_and_mul():
    silu = lambda z: z / (1 + math.exp(-z))
    one = torch.eye(2)
    # gate = [1, 2], up = [3, 4]  (activation.rs:60-70), through identity matrices
    x = torch.tensor([[1.0, 2.0]])
    up_w = torch.tensor([[3.0, 0.0], [0.0, 2.0]])
    out = P.swiglu(x, one, up_w, one, torch.float32)
    assert torch.allclose(out, torch.tensor([[silu(1.0) * 3.0, silu(2.0) * 4.0]]), atol=1e-6)
    z = P.swiglu(torch.tensor([[0.0, -50.0]]), one, one * 99, one, torch.float32)
    assert z.abs().max() < 1e-6                   # activation.rs:72-88


def test_attention_single_key_and_uniform():
    q = torch.randn(3, 2, 4)
    k = torch.zeros(3, 1, 4)
    v = torch.arange(12.0).reshape(3, 1, 4)
    out = P.attention(q, k, v, torch.arange(3), None, torch.float32).reshape(3, 2, 4)
    # all scores equal -> the mean of the visible values; first token sees only itself
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[2, 1], v[:, 0].mean(0), atol=1e-6)
    outw = P.attention(q, k, v, torch.arange(3), 2, torch.float32).reshape(3, 2, 4)
    assert torch.allclose(outw[2, 0], v[1:, 0].mean(0), atol=1e-6)   # window 2: positions 1 and 2


def test_whole_model_runs_and_is_causal(plain_models):
    cfg, w = plain_models["B"]
    ids = list(range(1, 20))
    full = P.forward_logits(cfg, w, ids, torch.float32)
    part = P.forward_logits(cfg, w, ids[:11], torch.float32)
    assert full.shape == (19, cfg["vocab_size"])
    assert torch.allclose(full[:11], part, atol=1e-5)


def test_window_changes_only_far_tokens(plain_models):
    cfg, w = plain_models["C"]
    ids = list(range(3, 63))
    a = P.forward_logits(cfg, w, ids, torch.float32)
    nocfg = dict(cfg, use_sliding_window=False)
    b = P.forward_logits(nocfg, w, ids, torch.float32)
    W = cfg["sliding_window"]
    assert torch.allclose(a[:W], b[:W], atol=1e-5)
    assert not torch.allclose(a[W + 8:], b[W + 8:], atol=1e-4)


# ------------------------------------------------------------------ sampler
def test_greedy_and_ties():
    assert S.sample_row([0.0, 5.0, 5.0, 1.0], 0.0, None, None, 1) == 1     # sampler.rs:293-305
    assert S.sample_row([0.0, 5.0, 7.0, 1.0], 1.0, 1, None, 1) == 2        # top_k 1 == greedy


def test_top_k_keeps_ties_and_top_p_cut():
    x, keep = S.surviving_mask(np.array([1.0, 3.0, 3.0, 2.0, 0.0], np.float32), 1.0, 2, None)
    assert keep.tolist() == [False, True, True, False, False]
    x, keep = S.surviving_mask(np.array([1.0, 3.0, 3.0, 3.0, 0.0], np.float32), 1.0, 2, None)
    assert keep.tolist() == [False, True, True, True, False]               # ties kept, sampler.rs:349-364
    probs = np.array([0.5, 0.3, 0.15, 0.05])
    x, keep = S.surviving_mask(np.log(probs).astype(np.float32), 1.0, None, 0.7)
    assert keep.tolist() == [True, True, False, False]                      # cumulative 0.5, 0.8 >= 0.7
    x, keep = S.surviving_mask(np.log(probs).astype(np.float32), 1.0, None, 0.85)
    assert keep.tolist() == [True, True, True, False]


def test_sampling_follows_the_distribution():
    probs = np.array([0.6, 0.25, 0.1, 0.05])
    logits = np.log(probs).astype(np.float32)
    draws = np.array([S.sample_row(logits, 1.0, None, None, key) for key in range(4000)])
    freq = np.bincount(draws, minlength=4) / 4000
    assert np.abs(freq - probs).max() < 0.03
    inside = {S.sample_row(logits, 1.0, 2, None, key) for key in range(200)}
    assert inside <= {0, 1}                                                 # sampler.rs: sampled in top-k


def test_penalties_once_per_distinct_token():
    out = S.apply_penalties(np.array([4.0, 4.0, 4.0], np.float32), [1, 1, 1, 2], 0.5, 0.25, 2.0)
    assert np.allclose(out, [4.0, 4.0 / 2 - 0.5 - 0.75, 4.0 / 2 - 0.5 - 0.25])   # sampler.rs:320-345
